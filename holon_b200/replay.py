"""Trace replay: feeds given token ids through the model step by step and writes logits. It samples nothing.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N [--page-size P]

Standard input brings one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step run as one batch through the engine's own step function, cache manager and kernels (the
ones generation uses; this file has no forward pass of its own). A request is admitted when its id first appears
and continues where it stopped; ids listed under `end` give back what they hold after the step. For a step that
wants logits, `DIR/<step>.f32` receives them as little-endian float32 [wanted, vocab], in the order of the entries
and of each entry's `want`. After every step a line `done <step>` is printed and flushed. The cache pool holds
`--max-tokens` tokens, each live request's count rounded up to whole pages of `--page-size` tokens (64 unless given),
so pages are used again.

The reference has no such program; the nearest are its teacher-forced scoring and its per-step snapshot trace
(judge/holon_judge/engine.py:49-80, judge/holon_judge/snapshot.py:59-99).
"""
from __future__ import annotations

import argparse
import json
import pathlib
import sys

PAGE_SIZE = 64
MAX_LIVE = 16


class Replayer:
    def __init__(self, model: str, dtype: str, max_tokens: int, device="cuda:0", kernels=None,
                 page_size: int = PAGE_SIZE) -> None:
        from .engine import build
        from .weights import SafetensorsSource
        pages = max(1, -(-max_tokens // page_size))
        self.built = build(SafetensorsSource(model), dtype=dtype, device=device, kernels=kernels, page_size=page_size,
                           max_seqs=MAX_LIVE, max_model_len=pages * page_size, max_step_tokens=pages * page_size,
                           pages=pages)
        self.slots: dict[str, int] = {}

    def step(self, record: dict):
        """Runs one step; returns the logits tensor [wanted, vocab] (32-bit) or None."""
        from .engine import StepEntry
        cache, entries = self.built.cache, []
        for e in record.get("entries", []):
            rid, tokens = str(e["id"]), [int(t) for t in e["tokens"]]
            if rid not in self.slots:
                slot = cache.admit()
                if slot is None:
                    raise RuntimeError(f"step {record.get('step')}: more than {MAX_LIVE} live requests")
                self.slots[rid] = slot
            slot = self.slots[rid]
            start = int(cache.computed[slot])
            if not cache.reserve(slot, start + len(tokens)):
                raise RuntimeError(f"step {record.get('step')}: request {rid!r} needs {start + len(tokens)} tokens; the "
                                   f"pool of --max-tokens has {cache.free_tokens()} free")
            entries.append(StepEntry(slot, tokens, start, [int(w) for w in e.get("want", [])]))
        logits = self.built.runner.step(entries) if entries else None
        for rid in record.get("end", []):
            slot = self.slots.pop(str(rid), None)
            if slot is not None:
                cache.release(slot)
        return logits


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=("bfloat16", "float32"),
                    help="bfloat16: the serving kernels; float32: everything in true 32-bit")
    ap.add_argument("--out", required=True, help="folder that receives <step>.f32")
    ap.add_argument("--max-tokens", required=True, type=int,
                    help="the most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    ap.add_argument("--page-size", type=int, default=PAGE_SIZE, help="tokens per page of the cache (default: 64)")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)
    if args.page_size < 1:
        ap.error("--page-size must be at least 1")
    out = pathlib.Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    import torch
    with torch.inference_mode():
        replayer = Replayer(args.model, args.dtype, args.max_tokens, args.device, page_size=args.page_size)
        for line in sys.stdin:
            line = line.strip()
            if not line:
                continue
            record = json.loads(line)
            logits = replayer.step(record)
            if logits is not None and logits.shape[0]:
                (out / f"{record['step']}.f32").write_bytes(logits.float().cpu().contiguous().numpy().astype("<f4").tobytes())
            else:
                torch.cuda.synchronize()
            print(f"done {record['step']}", flush=True)
    return 0
