"""Replay on the GPU, in true 32-bit and in bfloat16, against the plain implementation: whole requests; most of a
request in one step and its last 32 tokens one by one; portions of changing size down to two tokens; up to four live
requests mixed, portions of some beside decoded tokens of others, in a pool so small that pages are used again; long
decoding; the first tokens of a sequence; and the command-line program itself."""
from __future__ import annotations

import json
import pathlib
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from helpers import make_folder, random_prompt
from holon_b200.replay import Replayer
from replay_tools import TOLERANCE, compare, exact_and_rounded, mixed_trace, portions, run

pytestmark = pytest.mark.gpu
ROOT = pathlib.Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module", params=["a", "b", "c"])
def model(request, tmp_path_factory):
    folder = make_folder(tmp_path_factory.mktemp("models"), request.param)
    config, weights = plain.read_folder(folder)
    lengths = (70, 133, 37, 96)
    prompts = {f"r{i}": random_prompt(config["vocab_size"], n, 40 + i) for i, n in enumerate(lengths)}
    want = {rid: exact_and_rounded(config, weights, ids) for rid, ids in prompts.items()}
    return folder, config, prompts, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_then_tail_then_portions(model, dtype):
    folder, config, prompts, want = model
    r = Replayer(str(folder), dtype, max_tokens=192)
    # each request alone and whole
    got = run(r, [([(rid, ids)], [rid]) for rid, ids in prompts.items()])
    assert len(got) == sum(map(len, prompts.values()))
    compare(got, want, dtype)
    # most of it in one step, the last 32 tokens one by one
    steps = []
    for rid, ids in prompts.items():
        cut = len(ids) - 32
        steps.append(([(rid, ids[:cut])], []))
        steps += [([(rid, [t])], [rid] if i == 31 else []) for i, t in enumerate(ids[cut:])]
    compare(run(r, steps), want, dtype)
    # portions of changing size, down to two tokens
    steps = []
    for rid, ids in prompts.items():
        parts = portions(ids, [7, 2, 19, 3, 2, 64, 5])
        steps += [([(rid, p)], [rid] if i == len(parts) - 1 else []) for i, p in enumerate(parts)]
    compare(run(r, steps), want, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_requests_in_a_small_pool(model, dtype):
    """Four requests live at once in 448 tokens of pool (7 pages of 64): r1, r2 and r3 prefill in portions while r0
    decodes; when r0 ends, r3 grows into a page that r0 gave back."""
    folder, config, prompts, want = model
    r = Replayer(str(folder), dtype, max_tokens=448)
    steps = mixed_trace(prompts)
    got = run(r, steps)
    assert len(got) == sum(map(len, prompts.values()))
    compare(got, want, dtype)
    assert not r.built.cache.live


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(model, dtype):
    folder, config, _, _ = model
    _, weights = plain.read_folder(folder)
    ids = random_prompt(config["vocab_size"], 300, 77)
    want = {"x": exact_and_rounded(config, weights, ids)}
    r = Replayer(str(folder), dtype, max_tokens=320)
    got = run(r, [([("x", [t])], ["x"] if i == len(ids) - 1 else []) for i, t in enumerate(ids)])   # all one by one
    compare(got, want, dtype)
    first = {(rid, pos): row for (rid, pos), row in got.items() if pos < 4}
    assert len(first) == 4
    compare(first, want, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page_size", [4, 16])
def test_small_pages(model, dtype, page_size):
    """Pages of 4 and of 16 tokens: portions that end inside, at and across page edges, four live requests in a pool
    with one page to spare, pages given back and used again. (The tensor-core attention kernels take any page size;
    only their TMA-fed variants want multiples of 64.)"""
    folder, config, prompts, want = model
    live = sum(-(-len(ids) // page_size) * page_size for ids in list(prompts.values())[:3]) + page_size
    r = Replayer(str(folder), dtype, max_tokens=live, page_size=page_size)
    p = prompts
    steps, at = [], {rid: 0 for rid in p}
    sizes = {"r0": [page_size, 1, page_size - 1, 2, 3 * page_size + 1], "r1": [2 * page_size + 3, 1, 1, page_size, 7],
             "r2": [1, 2, page_size + 1], "r3": [5, page_size, 2]}
    turn = 0
    while any(at[rid] < len(p[rid]) for rid in ("r0", "r1", "r2")):
        entries, end = [], []
        for rid in ("r0", "r1", "r2"):
            if at[rid] < len(p[rid]):
                n = min(sizes[rid][turn % len(sizes[rid])], len(p[rid]) - at[rid])
                entries.append((rid, p[rid][at[rid]:at[rid] + n]))
                at[rid] += n
                if at[rid] == len(p[rid]):
                    end.append(rid)
        steps.append((entries, end))
        turn += 1
    while at["r3"] < len(p["r3"]):                                   # r3 runs in pages the others gave back
        n = min(sizes["r3"][turn % 3], len(p["r3"]) - at["r3"])
        steps.append(([("r3", p["r3"][at["r3"]:at["r3"] + n])], ["r3"] if at["r3"] + n == len(p["r3"]) else []))
        at["r3"] += n
        turn += 1
    got = run(r, steps)
    assert len(got) == sum(map(len, prompts.values()))
    compare(got, want, dtype)
    assert not r.built.cache.live


def test_command_line_program(model, tmp_path):
    folder, config, prompts, want = model
    ids = prompts["r2"]
    lines = [{"step": 0, "entries": [{"id": "a", "tokens": ids[:20], "want": [0, 19]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": ids[20:22], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": ids[22:], "want": [len(ids) - 23]},
                                     {"id": "b", "tokens": ids[:5], "want": [4]}], "end": ["a", "b"]}]
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32",
                           "--out", str(out), "--max-tokens", "128", "--page-size", "16"],
                          input="\n".join(map(json.dumps, lines)) + "\n",
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr
    assert proc.stdout.split() == ["done", "0", "done", "1", "done", "2"]
    assert not (out / "1.f32").exists()
    v = config["vocab_size"]
    s0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, v))
    s2 = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(-1, v))
    assert s0.shape[0] == 2 and s2.shape[0] == 2
    for row, pos in ((s0[0], 0), (s0[1], 19), (s2[0], len(ids) - 1), (s2[1], 4)):
        assert float((row - want["r2"][0][pos]).abs().max()) <= TOLERANCE


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_weights_stored_in_32_bits(tmp_path, dtype):
    """A folder whose tensors are all stored as float32. The float32 engine uses them as they are. The bfloat16 engine
    keeps products' weights and the embedding in bfloat16 and the norm weights in 32 bits (its norm and rotation
    kernels take both), so the yardstick is the plain implementation on weights rounded the same way."""
    folder = make_folder(tmp_path, "b", dtype=torch.float32)
    config, weights = plain.read_folder(folder)
    if dtype == "bfloat16":
        weights = {k: (v if k.endswith("norm.weight") or k.endswith("layernorm.weight") else v.bfloat16().float())
                   for k, v in weights.items()}
    ids = random_prompt(config["vocab_size"], 90, 3)
    want = {"x": exact_and_rounded(config, weights, ids)}
    r = Replayer(str(folder), dtype, max_tokens=128)
    norms = [p.tensor.dtype for name, p in r.built.model.params() if name.endswith("norm.weight")]
    assert set(norms) == {torch.float32}
    got = run(r, [([("x", ids[:61])], []), ([("x", ids[61:63])], [])] + [([("x", [t])], []) for t in ids[63:]])
    compare(got, want, dtype)


@pytest.mark.parametrize("kind", ["tickets", "ring"])
def test_products_chained_in_one_kernel_through_the_engine(model, monkeypatch, kind):
    """With HOLON_B200_CHAIN set the kernel table queues a decode step's consecutive products (o_proj, gate/up, down,
    the next layer's QKV) and runs them in one launch: the mixed trace (steps of up to 16 tokens take that path, larger
    ones the usual one) must give the same logits as ever."""
    from holon_b200.kernels import load_kernels
    folder, config, prompts, want = model
    kernels = load_kernels("cuda:0")
    monkeypatch.setattr(kernels, "chain", kind)
    before = kernels.chain_launches
    r = Replayer(str(folder), "bfloat16", max_tokens=448)
    got = run(r, mixed_trace(prompts))
    assert kernels.chain_launches - before > 50 and not kernels._pending
    compare(got, want, "bfloat16")
    assert kernels.tcgen05_status() == 0


def test_fused_products_of_17_to_64_rows_through_the_engine(model, monkeypatch):
    """With HOLON_B200_MID=all steps of 17 to 64 tokens keep the q/k norm, rotation and cache write, SwiGLU and the
    residual sum with the next norm inside their products (csrc/gemm_mid.cu): the mixed trace, whose steps bring 1 to
    70 tokens, must give the same logits as ever."""
    from holon_b200.kernels import load_kernels
    folder, config, prompts, want = model
    kernels = load_kernels("cuda:0")
    monkeypatch.setattr(kernels, "mid_mode", "all")
    before = kernels.mid_launches
    r = Replayer(str(folder), "bfloat16", max_tokens=448)
    steps = mixed_trace(prompts)
    sizes = [sum(len(tokens) for _, tokens in entries) for entries, _ in steps]
    assert any(16 < n <= 64 for n in sizes), sizes
    got = run(r, steps)
    # (per layer SwiGLU's product and the products that end the mixer and the feed-forward; the attention's first
    # product too where the head size is one its epilogue takes)
    assert kernels.mid_launches - before >= 2 * config["num_hidden_layers"] * sum(16 < n <= 64 for n in sizes)
    compare(got, want, "bfloat16")
    assert kernels.tcgen05_status() == 0
