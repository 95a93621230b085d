"""Measures decode and prefill throughput at Qwen3-8B sizes with random weights on one B200, for this engine and,
with `--impl reference`, for mxinO/holon itself through the same loops.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of the whole batch. The default run: the layer sizes of Qwen3-8B (36 layers, hidden
4096, 32 query heads, 8 KV heads, head size 128, intermediate 12288, vocabulary 151936), bfloat16, batch 8, each
request ending at a context of 8,192 tokens. It prints ONE JSON line:

  value            decoded tokens per second, timed on the device with CUDA events around exactly K steps of the
                   engine's `step()`, after W untimed ones
  e2e              the same through the public streaming calls a user makes (`add` with host token lists, `step`,
                   `has_work`; token ids back on the host with every step): tokens that arrive after every request's
                   first token, over the wall time from that moment to the last arrival, as the reference's own
                   benchmark takes it (bench/llama_bench.py:90-128). Every step copies its inputs from pinned host
                   memory and its tokens back; the bytes per step are counted from the tensors copied
  prefill          one prompt of 2,048 tokens: tokens per second, milliseconds, flops / time / bf16 peak
  roofline         the decode step's bytes (every weight once, the live requests' cache) / its time against the
                   measured copy bandwidth
  points           decode tokens per second at batch 1 and 64, and at batch 1, 8 and 64 with 2,048-token prompts and
                   256 decoded tokens; `point_rooflines` gives each point's bytes, milliseconds a step and fraction
  kernels          every kernel of one decode layer and of one prefill layer alone, with CUDA events: microseconds,
                   bytes or flops, and the fraction of the copy bandwidth or of the bf16 peak (this engine only)
  clocks           SM clocks sampled with nvidia-smi during the timed steps

Every decode step reads 15 GB of weights and the requests' cache, far more than the 126 MB L2, so consecutive steps
cannot reuse cached data ("l2": "inputs larger than L2"). Peaks come from MEASURED_PEAKS.json beside this file if it
is there, else from an earlier measurement of a B200 (6.65 TB/s copy, 1.59 PFLOP/s bf16).

`--impl reference` runs the unmodified reference from baseline/_ref (see baseline/install_ref.py) through its own
`Engine`, `EngineConfig` and `SamplingParams`, on the same weights (written once to a temporary model folder), the
same prompts, batch, context, K and W, and prints the same keys with "impl": "reference".
"""
from __future__ import annotations

import argparse
import json
import pathlib
import statistics
import subprocess
import sys
import time

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=36, hidden_size=4096, num_attention_heads=32,
                num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=151936, rope_theta=1000000.0,
                rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=40960)
FULL_LAYERS = QWEN3_8B["num_hidden_layers"]
# The other two sizes the benchmark's configurations name, for `--only sizes --sizes ...` (their own workloads).
QWEN3_06B = dict(QWEN3_8B, num_hidden_layers=28, hidden_size=1024, num_attention_heads=16, intermediate_size=3072,
                 tie_word_embeddings=True)
QWEN3_32B = dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, intermediate_size=25600)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def _find_number(data, key: str):
    """The first number stored under `key` anywhere in a nested JSON value (a dict under the key: its "value")."""
    if isinstance(data, dict):
        if key in data:
            v = data[key]
            if isinstance(v, dict):
                v = v.get("value", v.get("median", v.get("max")))
            if isinstance(v, (int, float)) and not isinstance(v, bool):
                return float(v)
        for v in data.values():
            found = _find_number(v, key)
            if found is not None:
                return found
    elif isinstance(data, list):
        for v in data:
            found = _find_number(v, key)
            if found is not None:
                return found
    return None


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            data = json.loads(path.read_text())
            hbm, flops = _find_number(data, "hbm_gbs"), _find_number(data, "bf16_tflops")
            if hbm and flops:
                return {"hbm_gbs": hbm, "bf16_tflops": flops}, "measured"
        except (ValueError, OSError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class Clocks:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed steps run."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.proc, self.marked = None, 0.0

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu=timestamp,{self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def mark(self) -> None:
        """Samples taken before this moment (the warm-up) are left out."""
        self.marked = time.time()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        out, _ = self.proc.communicate()
        sm, top, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.splitlines():
            cells = [c.strip() for c in line.split(",")]
            if len(cells) < 7:
                continue
            try:
                stamp = time.mktime(time.strptime(cells[0].split(".")[0], "%Y/%m/%d %H:%M:%S"))
            except ValueError:
                stamp = self.marked
            cells = cells[1:]
            if not cells[0].isdigit() or stamp + 1 < self.marked:
                continue
            sm.append(int(cells[0]))
            top.append(int(cells[1]))
            reasons.update(n for n, c in zip(names, cells[2:6]) if c.lower().startswith("active"))
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(top) if top else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def model_numbers(cfg: dict, layers: int) -> dict:
    """Parameter bytes a decode step reads and flops per token, from the configuration."""
    h, d, hq, hkv, inter, v = (cfg[k] for k in ("hidden_size", "head_dim", "num_attention_heads",
                                                "num_key_value_heads", "intermediate_size", "vocab_size"))
    per_layer = (hq + 2 * hkv) * d * h + hq * d * h + 3 * inter * h
    linear = layers * per_layer + v * h                              # the head reads its table once; the embedding rows are few
    return {"weight_bytes": 2 * linear, "linear_params": linear, "kv_bytes_per_token": layers * 2 * hkv * d * 2,
            "attn_flops_per_pair": 4 * hq * d * layers}


def prompts_of(vocab: int, batch: int, length: int, seed: int) -> list[list[int]]:
    import torch
    g = torch.Generator().manual_seed(seed)
    return torch.randint(1000, vocab // 2, (batch, length), generator=g).tolist()


class Arm:
    """An engine under the benchmark's loops. This engine and the reference answer the same calls (`add`, `step`,
    `has_work`, `abort`, `drain`: the reference's names, core/holon/core/engine.py:332-524), so one set of loops times
    both; what differs is gathered here."""

    impl = "holon_b200"

    def __init__(self, engine) -> None:
        self.engine = engine

    def params(self, max_tokens: int):
        from holon_b200.engine import SamplingParams
        return SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=True)

    @property
    def sched(self):
        return self.engine.scheduler

    @property
    def vocab(self) -> int:
        return self.engine.built.model.spec.vocab

    def counters(self):
        """(bytes copied to the device, bytes copied back, kernels of this package launched) so far."""
        e = self.engine
        return e.h2d_bytes, e.d2h_bytes, e.launches()


class ReferenceArm(Arm):
    impl = "reference"

    def params(self, max_tokens: int):
        from holon.api import SamplingParams
        return SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=True)

    @property
    def sched(self):
        return self.engine.sched

    @property
    def vocab(self) -> int:
        return self.engine.spec.vocab

    def counters(self):
        return None                                                  # the reference does not count its copies


def decode_run(arm: Arm, batch: int, context: int, steps: int, warmup: int, seed: int, clocks: Clocks | None = None) -> dict:
    """`batch` equal prompts, prefilled (untimed) so that the last timed step ends at `context` tokens; then `warmup`
    untimed and `steps` timed decode steps through the engine's `step`."""
    import torch
    engine = arm.engine
    prompt_len = context - (steps + warmup) - 1
    params = arm.params(steps + warmup + 1)
    rids = [engine.add(p, params) for p in prompts_of(arm.vocab, batch, prompt_len, seed)]
    while arm.sched.waiting:                                         # prefill, in portions under the token budget
        engine.step()
    assert len(arm.sched.running) == batch
    if clocks:
        clocks.start()                                              # (nvidia-smi needs a moment before its first sample)
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    if clocks:
        clocks.mark()
    before = arm.counters()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    start.record()
    produced = 0
    for _ in range(steps):
        produced += sum(len(d.token_ids) for d in engine.step())
    end.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    device_ms = start.elapsed_time(end)
    clock = clocks.stop() if clocks else None
    assert produced == batch * steps, (produced, batch, steps)
    out = {"device_ms": device_ms, "wall_ms": wall * 1e3, "tokens": produced, "mean_context": context - (steps + 1) / 2,
           "clocks": clock, "h2d_bytes_per_step": None, "d2h_bytes_per_step": None, "launches": None}
    if before is not None:
        after = arm.counters()
        out |= {"h2d_bytes_per_step": (after[0] - before[0]) // steps, "d2h_bytes_per_step": (after[1] - before[1]) // steps,
                "launches": after[2] - before[2]}
    for rid in rids:
        engine.abort(rid)
    engine.drain()
    return out


def stream_run(arm: Arm, batch: int, context: int, steps: int, warmup: int, seed: int) -> dict:
    """Decode throughput end to end, through the calls a user streams with: host token lists go in with `add`, every
    `step` brings the new token ids back to the host, and the wall clock is read when they arrive (the reference's
    benchmark times the same loop: bench/llama_bench.py:35-49, 118-121). Each request generates `warmup` + `steps` + 1
    tokens and ends at `context`. Two passes with fresh prompts:

    - `after_prefill`: `batch * steps` tokens over the time from the moment every request has its first token to the
      arrival of the `steps`-th token after it: decoding straight after the prompts' computation, which runs under the
      power cap and leaves the SM clocks low for the first tens of milliseconds (`gaps_ms` shows the ramp);
    - `value`: the protocol of the device-timed run, by wall clock: when every request has its first token the clock
      sampler is started, then `warmup` arrivals pass untimed and `batch * steps` tokens are timed from the `warmup`-th
      arrival to the last; the clocks sampled meanwhile are returned."""
    import torch
    engine, out = arm.engine, {}
    prompt_len = context - (steps + warmup) - 1
    for sampled in (True, False):                                    # (the timed protocol first: it then follows the same
                                                                     # history as the device-timed run, one prompt phase, not two)
        prompts = prompts_of(arm.vocab, batch, prompt_len, seed + sampled)
        params = arm.params(steps + warmup + 1)
        clocks = Clocks() if sampled else None
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        rids = [engine.add(p, params) for p in prompts]
        first, moments, began = {}, [], None
        while engine.has_work():
            deltas = engine.step()
            now = time.perf_counter() - t0
            arrived = [d for d in deltas if d.token_ids]
            for d in arrived:
                first.setdefault(d.rid, now)
            if began is not None and arrived:
                moments.append(now)
            if began is None and len(first) == len(rids):
                began = now
                if clocks:
                    clocks.start()                                   # (every sample from here on lies in the decode part)
        clock = clocks.stop() if clocks else None
        assert began is not None and len(moments) == steps + warmup, (began, len(moments))
        if sampled:
            seconds = moments[warmup + steps - 1] - moments[warmup - 1]
            out |= {"value": batch * steps / seconds, "seconds": seconds, "tokens": batch * steps, "clocks": clock}
        else:
            seconds = moments[steps - 1] - began
            out["after_prefill"] = {"value": round(batch * steps / seconds, 1), "seconds": round(seconds, 5),
                                    "gaps_ms": [round((b - a) * 1e3, 2) for a, b in zip([began] + moments, moments)]}
    return out


def prefill_run(arm: Arm, tokens: int, repeats: int, seed: int) -> float:
    """Milliseconds (device, best of `repeats`) of one step that computes a whole prompt of `tokens` tokens and samples
    its first token."""
    import torch
    engine, best = arm.engine, float("inf")
    for i in range(repeats + 1):                                     # the first one is a warm-up
        engine.add(prompts_of(arm.vocab, 1, tokens, seed + i)[0], arm.params(1))
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        deltas = engine.step() + engine.drain()                      # the step, and its token read back
        end.record()
        torch.cuda.synchronize()
        assert len(deltas) == 1 and deltas[0].finish_reason == "length"
        if i:
            best = min(best, start.elapsed_time(end))
    return best


def long_prompt_run(args) -> dict:
    """Time to the first token of a 30,000-token prompt that arrives while three requests decode (prompt portions of
    up to 2,048 tokens beside their decode rows): the reference's long-prompt case (docs/dev/release.md:3103)."""
    import torch
    from holon_b200.engine import Engine, EngineConfig, SamplingParams
    from holon_b200.weights import RandomSource
    cfg = dict(QWEN3_8B, num_hidden_layers=args.layers)
    engine = Engine(EngineConfig(model="random weights, seed 2", device="cuda:0", dtype="bfloat16", page_size=64,
                                 max_seqs=8, max_model_len=32768, max_step_tokens=4096, chunk_with_decode=2048, seed=0, prefix_cache=False),
                    source=RandomSource(cfg, seed=2, device="cuda:0"))
    vocab, best = engine.built.model.spec.vocab, float("inf")
    streams = SamplingParams(temperature=0.0, max_tokens=400, ignore_eos=True)
    for rep in range(3):                                             # the first one is a warm-up
        for prompt in prompts_of(vocab, 3, 256, 70 + rep):
            engine.add(prompt, streams)
        for _ in range(20):
            engine.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        rid = engine.add(prompts_of(vocab, 1, 30000, 80 + rep)[0], SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True))
        first, steps = None, 0
        while first is None:
            steps += 1
            if any(d.rid == rid for d in engine.step()):
                first = time.perf_counter() - t0
        if rep:
            best = min(best, first)
        for r in list(engine.requests):
            engine.abort(r)
        engine.drain()
    return {"only": "long_prompt", "layers": args.layers, "prompt_tokens": 30000, "streams": 3, "ttft_ms": round(best * 1e3, 1),
            "prompt_tokens_per_s": round(30000 / best, 1), "steps": steps}


def sizes_run(args) -> dict:
    """The workloads of the two other configurations: Qwen3-32B sizes (decode at batch 1 and 64 over 4,096-token
    prompts, prefill of one 8,192-token prompt, context 16,384) and Qwen3-0.6B sizes (32 requests with prompts uniform
    in [16, 4096] tokens, prompt portions of 512 beside the decode rows, 128 tokens each, through `Engine.generate`)."""
    import random
    import torch
    from holon_b200.engine import Engine, EngineConfig, SamplingParams
    from holon_b200.weights import RandomSource
    peak, peak_kind = peaks()
    out = {"only": "sizes", "sizes": args.sizes, "peaks": peak_kind}
    if args.sizes == "32b":
        cfg, seed = dict(QWEN3_32B), 4
        engine = Engine(EngineConfig(model="random weights, seed 4", device="cuda:0", dtype="bfloat16", page_size=64,
                                     max_seqs=64, max_model_len=16384, max_step_tokens=8192, seed=0, prefix_cache=False),
                        source=RandomSource(cfg, seed=seed, device="cuda:0"))
        numbers = model_numbers(cfg, cfg["num_hidden_layers"])
        tokens = 8192
        ms = prefill_run(Arm(engine), tokens, repeats=2, seed=100)
        flops = 2 * numbers["linear_params"] * tokens - 2 * cfg["vocab_size"] * cfg["hidden_size"] * (tokens - 1) \
            + numbers["attn_flops_per_pair"] * tokens * (tokens + 1) / 2
        out["prefill"] = {"value": round(tokens / ms * 1e3, 1), "tokens": tokens, "ms": round(ms, 2),
                          "frac": round(flops / (ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4)}
        steps = max(8, min(args.steps, 64))
        for b in (1, 64):
            r = decode_run(Arm(engine), b, 4096 + steps + args.warmup + 1, steps, args.warmup, seed=11 + b)
            ms_step = r["device_ms"] / steps
            moved = numbers["weight_bytes"] + b * r["mean_context"] * numbers["kv_bytes_per_token"]
            out[f"decode_b{b}"] = {"value": round(r["tokens"] / r["device_ms"] * 1e3, 1), "ms_per_step": round(ms_step, 3),
                                   "hbm_frac": round(moved / (ms_step * 1e-3) / 1e9 / peak["hbm_gbs"], 4)}
    else:
        cfg, seed = dict(QWEN3_06B), 3
        engine = Engine(EngineConfig(model="random weights, seed 3", device="cuda:0", dtype="bfloat16", page_size=64,
                                     max_seqs=32, max_model_len=4352, max_step_tokens=4096, chunk_with_decode=512, seed=0, prefix_cache=False),
                        source=RandomSource(cfg, seed=seed, device="cuda:0"))
        rng = random.Random(5)
        prompts = [[rng.randrange(cfg["vocab_size"]) for _ in range(rng.randint(16, 4096))] for _ in range(32)]
        params = SamplingParams(temperature=0.0, max_tokens=128, ignore_eos=True)
        best = float("inf")
        for rep in range(3):                                         # the first one is a warm-up
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            got = engine.generate(prompts, params)
            torch.cuda.synchronize()
            if rep:
                best = min(best, time.perf_counter() - t0)
        n_prompt, n_out = sum(map(len, prompts)), sum(map(len, got))
        out["serve"] = {"requests": 32, "prompt_tokens": n_prompt, "generated_tokens": n_out, "seconds": round(best, 4),
                        "generated_tokens_per_s": round(n_out / best, 1), "all_tokens_per_s": round((n_prompt + n_out) / best, 1),
                        "chunk_with_decode": 512, "stats": engine.stats()}
        engine.close()
        del engine                                                   # (its cache pool took the free memory)
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        engine = Engine(EngineConfig(model="random weights, seed 3", device="cuda:0", dtype="bfloat16", page_size=64,
                                     max_seqs=32, max_model_len=4352, max_step_tokens=4096, seed=0, prefix_cache=False),
                        source=RandomSource(cfg, seed=seed, device="cuda:0"))
        numbers = model_numbers(cfg, cfg["num_hidden_layers"])
        steps = max(8, min(args.steps, 64))
        for b in (1, 32):
            r = decode_run(Arm(engine), b, 2048 + steps + args.warmup + 1, steps, args.warmup, seed=11 + b)
            ms_step = r["device_ms"] / steps
            moved = numbers["weight_bytes"] + b * r["mean_context"] * numbers["kv_bytes_per_token"]
            out[f"decode_b{b}"] = {"value": round(r["tokens"] / r["device_ms"] * 1e3, 1), "ms_per_step": round(ms_step, 3),
                                   "hbm_frac": round(moved / (ms_step * 1e-3) / 1e9 / peak["hbm_gbs"], 4)}
    out["config"] = {k: cfg[k] for k in ("num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads",
                                         "head_dim", "intermediate_size", "vocab_size", "tie_word_embeddings")}
    return out


def shared_prompt_run(args) -> dict:
    """16 requests whose prompts share their first 2,048 tokens (64 tokens of their own follow), 32 tokens generated
    each, through `Engine.generate`, with the prefix cache and without it: seconds for all of them, second pass (the
    first pass of the engine with the cache leaves the shared pages behind, as a system prompt does in serving)."""
    import gc
    import torch
    from holon_b200.engine import Engine, EngineConfig, SamplingParams
    from holon_b200.weights import RandomSource
    cfg = dict(QWEN3_8B, num_hidden_layers=args.layers)
    out = {"only": "shared_prompt", "layers": args.layers, "requests": 16, "shared_tokens": 2048, "own_tokens": 64,
           "generated_each": 32}
    params = SamplingParams(temperature=0.0, max_tokens=32, ignore_eos=True)
    for cached in (True, False):
        engine = Engine(EngineConfig(model="random weights, seed 2", device="cuda:0", dtype="bfloat16", page_size=64,
                                     max_seqs=16, max_model_len=4096, max_step_tokens=4096, chunk_with_decode=1024,
                                     seed=0, prefix_cache=cached, memory_fraction=0.5),
                        source=RandomSource(cfg, seed=2, device="cuda:0"))
        vocab, times = engine.built.model.spec.vocab, []
        for rep in range(3):                                         # other tokens every pass: only passes of one engine
            stem = prompts_of(vocab, 1, 2048, 500)[0]                # share the stem
            prompts = [stem + tail for tail in prompts_of(vocab, 16, 64, 600 + rep)]
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            got = engine.generate(prompts, params)
            times.append(time.perf_counter() - t0)
            assert all(len(g) == 32 for g in got)
        stats = engine.stats()
        out["prefix_cache" if cached else "no_prefix_cache"] = {
            "first_pass_s": round(times[0], 4), "later_pass_s": round(min(times[1:]), 4),
            "prefix_hit_tokens": stats["prefix_hit_tokens"], "steps": stats["steps"]}
        engine.close()
        del engine
        gc.collect()
        torch.cuda.empty_cache()
    return out


def headline(arm: Arm, args, cfg: dict, engine_facts: dict) -> dict:
    """The benchmark's line for one engine: the loops above at the sizes of `cfg`."""
    context, batch = args.context, args.batch
    numbers = model_numbers(cfg, cfg["num_hidden_layers"])
    peak, peak_kind = peaks()
    prefill_tokens = 2048
    prefill_ms = prefill_run(arm, prefill_tokens, repeats=3, seed=100)
    prefill_flops = 2 * numbers["linear_params"] * prefill_tokens - 2 * cfg["vocab_size"] * cfg["hidden_size"] * (prefill_tokens - 1) \
        + numbers["attn_flops_per_pair"] * prefill_tokens * (prefill_tokens + 1) / 2
    clocks = Clocks()
    main = decode_run(arm, batch, context, args.steps, args.warmup, seed=7, clocks=clocks)
    e2e = stream_run(arm, batch, context, args.steps, args.warmup, seed=31)

    def roofline_of(run: dict, rows: int, steps: int) -> dict:
        ms = run["device_ms"] / steps
        moved = numbers["weight_bytes"] + rows * run["mean_context"] * numbers["kv_bytes_per_token"]
        achieved = moved / (ms * 1e-3) / 1e9
        return {"gb": round(moved / 1e9, 3), "ms_per_step": round(ms, 4), "achieved": round(achieved, 1),
                "frac": round(achieved / peak["hbm_gbs"], 4), "mean_context": run["mean_context"]}

    points, point_rooflines = {}, {}
    few = max(8, min(args.steps, 64))
    workloads = [(f"decode_b{b}", b, context, few) for b in (1, 64)] if not args.no_points else []
    # the same with 2,048-token prompts and 256 decoded tokens a request: the steps timed are the last ones of the 256
    workloads += [(f"decode_b{b}_prompt2048", b, 2048 + 256, min(256 - args.warmup, max(8, args.steps)))
                  for b in (1, 8, 64)] if not args.no_points else []
    for name, b, ctx, steps in workloads:
        r = decode_run(arm, b, ctx, steps, args.warmup, seed=11 + b + ctx)
        points[name] = round(r["tokens"] / r["device_ms"] * 1e3, 1)
        point_rooflines[name] = roofline_of(r, b, steps)
    ms_per_step = main["device_ms"] / args.steps
    main_roofline = roofline_of(main, batch, args.steps)
    return {
        "metric": f"decode tok/s at batch {batch} (Qwen3-8B bf16, context {context}); points: batch 1/64 there, and batch "
                  "1/8/64 with 2,048-token prompts + 256 decoded; prefill of 2,048 tokens",
        "value": round(main["tokens"] / main["device_ms"] * 1e3, 1), "unit": "tok/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: uniform random token ids, seeded random weights", "impl": arm.impl,
        "config": {"model": "Qwen3-8B sizes", "layers": cfg["num_hidden_layers"], "layers_full": FULL_LAYERS,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": batch,
                   "seq_len": context, "parallelism": "single GPU", "l2": "inputs larger than L2", "peaks": peak_kind,
                   **engine_facts},
        "e2e": {"value": round(e2e["value"], 1), "unit": "tok/s", "h2d_bytes_per_step": main["h2d_bytes_per_step"],
                "d2h_bytes_per_step": main["d2h_bytes_per_step"],
                "method": "add / step / has_work with host token lists, wall clock at the arrivals: W arrivals untimed "
                          "after every request's first token, then batch * K tokens from the W-th arrival to the last",
                "tokens": e2e["tokens"], "seconds": round(e2e["seconds"], 5), "clocks": e2e["clocks"],
                "after_prefill": e2e["after_prefill"],
                "step_loop_wall_value": round(main["tokens"] / main["wall_ms"] * 1e3, 1)},
        "gpu_launches": main["launches"],
        "prefill": {"value": round(prefill_tokens / prefill_ms * 1e3, 1), "tokens": prefill_tokens,
                    "ms": round(prefill_ms, 3), "frac": round(prefill_flops / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": main_roofline["achieved"], "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": main_roofline["frac"], "gb": main_roofline["gb"]},
        "points": points, "point_rooflines": point_rooflines, "clocks": main["clocks"],
    }


def run_ours(args) -> dict:
    import torch
    from holon_b200.engine import Engine, EngineConfig
    from holon_b200.weights import RandomSource
    if args.only == "long_prompt":
        return long_prompt_run(args)
    if args.only == "sizes":
        return sizes_run(args)
    if args.only == "shared_prompt":
        return shared_prompt_run(args)
    cfg = dict(QWEN3_8B, num_hidden_layers=args.layers)
    context, batch = args.context, args.batch
    engine = Engine(EngineConfig(model="random weights, seed 2", device="cuda:0", dtype="bfloat16", page_size=64,
                                 max_seqs=64, max_model_len=context, max_step_tokens=8192, seed=0,
                                 memory_fraction=args.memory_fraction, prefix_cache=False),
                    source=RandomSource(cfg, seed=2, device="cuda:0"))
    print(f"bench: {engine.memory_report()}", file=sys.stderr, flush=True)
    arm = Arm(engine)
    if args.only == "decode":
        main = decode_run(arm, batch, context, args.steps, args.warmup, seed=7)
        return {"only": "decode", "layers": args.layers, "ms_per_step": round(main["device_ms"] / args.steps, 4)}
    if args.only == "prefill":
        return {"only": "prefill", "layers": args.layers, "ms": round(prefill_run(arm, 2048, repeats=3, seed=100), 3)}
    out = headline(arm, args, cfg, {"page_size": 64, "cuda_graphs": True, "overlap": engine.config.overlap,
                                    "prefix_cache": False, "gemm": engine.built.ctx.kernels.gemm})
    if not args.no_kernels:
        from holon_b200.kernels.microbench import layer_table
        peak, _ = peaks()
        out["kernels"] = layer_table(engine.built.ctx.kernels, cfg, batch, context, 2048, peak["hbm_gbs"], peak["bf16_tflops"])
    memory = engine.built.memory
    free, _ = torch.cuda.mem_get_info()
    out["memory"] = {"weights_gb": round(memory.weights / 1e9, 2), "cache_gb": round(memory.cache / 1e9, 2),
                     "activations_gb": round((memory.activations or 0) / 1e9, 3), "graphs_gb": round((memory.graphs or 0) / 1e9, 3),
                     "device_free_gb": round(free / 1e9, 2)}
    return out


def write_model_shards(cfg: dict, seed: int, folder: pathlib.Path, shard_bytes: int = 2 << 30) -> None:
    """config.json and the seeded random weights of `cfg` as safetensors shards of about `shard_bytes` each (the
    tensors are made on the GPU one by one, so the host never holds more than a shard)."""
    import torch
    from safetensors.torch import save_file
    from holon_b200.weights import RandomSource
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    shard, held, index = {}, 0, 0
    for name, tensor in RandomSource(cfg, seed=seed, device="cuda:0" if torch.cuda.is_available() else "cpu").tensors():
        shard[name] = tensor.cpu().contiguous()
        held += tensor.numel() * tensor.element_size()
        if held >= shard_bytes:
            save_file(shard, str(folder / f"model-{index:05d}.safetensors"))
            shard, held, index = {}, 0, index + 1
    if shard:
        save_file(shard, str(folder / f"model-{index:05d}.safetensors"))


def reference_plugins(ref: pathlib.Path, testing: bool = False):
    """The reference's plugin set, made from the `plugin.toml` manifests of its installed packages (its own
    `discover()` reads the same manifests through entry points, which a plain copy of the packages does not have).
    Its test-only plugins (CPU oracle kernels) stay out unless `testing`: a user's install has none of them."""
    from holon.api import Manifest
    from holon.core.plugins import Installed, PluginSet
    installed = {}
    for root in (ref / "holon_std", ref / "holon_plugins") + ((ref / "holon_testing",) if testing else ()):
        for toml in sorted(root.rglob("plugin.toml")):
            if "vendor" in toml.parts:
                continue
            manifest = Manifest.load(toml)
            installed[manifest.name] = Installed(manifest, ".".join(toml.parent.relative_to(root.parent).parts), toml.parent)
    return PluginSet(installed)


def run_reference(args) -> dict:
    """The reference arm: the unmodified reference from baseline/_ref, driven through its own `Engine`, `EngineConfig`
    and `SamplingParams` by the loops that time this engine, on the same weights, prompts and sizes. Nothing of this
    package is on its path but the weight files, written once to a temporary folder."""
    import shutil
    import tempfile
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "holon").is_dir():
        return {"impl": "reference", "unavailable": "baseline/_ref holds no copy of mxinO/holon: run "
                                                    "`python baseline/install_ref.py <checkout of the reference>` first"}
    if args.only != "all":
        return {"impl": "reference", "unavailable": f"--only {args.only} is a mode of this engine's arm alone"}
    folder = pathlib.Path(tempfile.mkdtemp(prefix="holon_b200_reference_model_"))
    engine = None
    stage = "importing the reference"
    try:
        import torch
        sys.path.insert(0, str(ref))
        from holon.core.engine import Engine, EngineConfig
        plugins = reference_plugins(ref)
        stage = "writing the model folder"
        cfg = dict(QWEN3_8B, num_hidden_layers=args.layers)
        write_model_shards(cfg, 2, folder)
        torch.cuda.empty_cache()
        stage = "building the reference's engine"
        engine = Engine(EngineConfig(model=str(folder), device="cuda:0", dtype=torch.bfloat16, max_seqs=64,
                                     max_model_len=args.context, max_step_tokens=8192, prefix_cache=False,
                                     memory_fraction=args.memory_fraction), plugins)
        stage = "running the reference's engine"
        facts = {"page_size": engine.cfg.page_size, "cuda_graphs": engine.cfg.cuda_graphs, "overlap": engine.cfg.overlap,
                 "prefix_cache": engine.cfg.prefix_cache}
        out = headline(ReferenceArm(engine), args, cfg, facts)     # (its own calls switch gradients off)
        selected = getattr(getattr(engine, "ctx", None), "selected", None)
        if selected:
            out["reference_kernels"] = {str(k): str(v) for k, v in dict(selected).items()}
        return out
    except Exception as e:                                           # what the reference raised here, in its own words
        text = " ".join(f"{type(e).__name__}: {e}".split())
        return {"impl": "reference", "unavailable": f"{stage} failed on this machine: {text[:600]}"}
    finally:
        try:
            if engine is not None:
                engine.close()
        except Exception:
            pass
        shutil.rmtree(folder, ignore_errors=True)


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers than the model has (both are reported)")
    ap.add_argument("--memory-fraction", type=float, default=0.9,
                    help="share of the free device memory for weights and cache pool; a run under a profiler that takes "
                         "several passes should hold a few GB only (e.g. 0.03 with --layers 4 --batch 8)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--only", default="all", choices=("all", "decode", "prefill", "long_prompt", "sizes", "shared_prompt"),
                    help="run one part only (for profiling a small case); the JSON line then lacks the other parts. "
                         "long_prompt: time to first token of a 30,000-token prompt behind three decoding requests; "
                         "sizes: the workloads of the Qwen3-32B and Qwen3-0.6B configurations (--sizes); "
                         "shared_prompt: 16 requests with a common 2,048-token beginning, with and without the prefix cache")
    ap.add_argument("--sizes", default="32b", choices=("32b", "0.6b"), help="with --only sizes: which configuration")
    ap.add_argument("--no-points", action="store_true", help="leave out the points at other batch sizes and contexts")
    ap.add_argument("--no-kernels", action="store_true", help="leave out the per-kernel table")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"this benchmark measures one GPU: --gpus {args.gpus} is not supported (holon_b200 is a single-GPU engine)")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        print(json.dumps(run_reference(args)))
        return 0
    import torch
    with torch.inference_mode():
        print(json.dumps(run_ours(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
