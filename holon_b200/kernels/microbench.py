"""Times single kernels of the kernel table with CUDA events, the L2 replaced between runs.

    python -m holon_b200.kernels.microbench decode_attention [--rows 8 64 1] [--context 8192] [--splits 4 6 13]
    python -m holon_b200.kernels.microbench gemm [--rows 2048] [--shapes qkv o gate_up down]
    python -m holon_b200.kernels.microbench prefill_attention [--rows 2048] [--context 2048]
    python -m holon_b200.kernels.microbench layer [--rows 8 1 16 64] [--context 8192]

`layer` times the kernels of a decode layer the way a step runs them: back to back inside a CUDA graph, each launch
on weights (or a cache) other than the launch before, several hundred MB in turn, so that nothing comes from the L2
and nothing of the host's pace or of an event's own cost is in the number.

Sizes default to Qwen3-8B's (32 query and 8 KV heads of 128, hidden 4096, intermediate 12288). `layer_table` times
every kernel of one decode layer and of one prefill layer the same way and sets each time against the bytes or the
flops the kernel has to move or do; `bench.py` prints it as its `kernels` block.
"""
from __future__ import annotations

import argparse
import ctypes
import math

import torch

from . import load_kernels
from ..engine.batch import Rows

SHAPES = {"qkv": (6144, 4096), "o": (4096, 4096), "gate_up": (24576, 4096), "down": (4096, 12288)}


def timed(fn, flush, runs: int = 6) -> float:
    """Microseconds of the fastest of `runs` calls, each after a buffer larger than the L2 was read through it
    (reading leaves clean lines; lines left dirty by a write would be written back during the timed kernel and
    take a share of its bandwidth)."""
    best = float("inf")
    for i in range(runs):
        if flush is not None:
            flush.view(torch.int32).sum()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        if i:
            best = min(best, start.elapsed_time(end) * 1e3)
    return best


def decode_attention(k, args) -> None:
    heads, kv_heads, d, page = 32, 8, 128, 64
    flush = torch.zeros(256 << 20, device=k.device, dtype=torch.uint8)
    for rows in args.rows:
        per = args.context // page
        kv = torch.randn(rows * per + 1, 2, kv_heads, page, d, device=k.device, dtype=torch.bfloat16)
        table = torch.arange(rows * per, device=k.device, dtype=torch.int32).view(rows, per).contiguous()
        q = torch.randn(rows, heads, d, device=k.device, dtype=torch.bfloat16)
        out = torch.empty_like(q)
        ar = torch.arange(rows + 1, device=k.device, dtype=torch.int32)
        batch = Rows(ar[:rows].contiguous(), ar, torch.full((rows,), args.context, device=k.device, dtype=torch.int32),
                     rows, rows, rows, 1, args.context)
        moved = rows * args.context * kv_heads * d * 2 * 2
        planned = k.decode_splits(rows, heads, kv_heads, args.context)
        call = lambda: k.paged_attention(out, q, kv, table, batch, 1 / math.sqrt(d), 0)   # noqa: E731
        k.decode_attention = "balanced"                    # (the rows keep a step's plan: forget it with every change)
        t = timed(call, flush)
        print(f"decode attention rows {rows} context {args.context} balanced: {t:7.1f} us  {moved / t / 1e6:5.2f} TB/s")
        k.decode_attention = "splits"
        batch.plan.clear()
        t = timed(call, flush)
        few = k.decode_cluster_splits(rows, heads, kv_heads, d, args.context, planned)
        print(f"decode attention rows {rows} context {args.context} as the kernel table runs it ("
              + (f"a cluster of {few} splits" if few else f"{planned} splits, merge kernel")
              + f"): {t:7.1f} us  {moved / t / 1e6:5.2f} TB/s")
        cluster, k.decode_cluster = k.decode_cluster, False
        for splits in (args.splits or [planned]):
            k._splits[(rows, heads, kv_heads, -(-args.context // 64), 64)] = splits
            t = timed(call, flush)
            print(f"decode attention rows {rows} context {args.context} splits {splits}, merge kernel: {t:7.1f} us  {moved / t / 1e6:5.2f} TB/s"
                  + ("  (the planner's choice)" if splits == planned else ""))
        k.decode_cluster = cluster
        for splits in args.cluster or []:                  # the cluster kernel itself, whatever the table would choose
            direct = lambda: k._call(                      # noqa: E731
                "hb_attention_decode_bf16_cluster", k._p(out), k._p(q), k._p(kv), k._i32(table, "table"), table.shape[1],
                k._i32(batch.row_slot, "slot"), k._i32(batch.query_start, "start"), k._i32(batch.kv_len, "len"), rows,
                heads, kv_heads, d, kv.shape[0], page, ctypes.c_float(1 / math.sqrt(d)), 0, splits)
            t = timed(direct, flush)
            print(f"decode attention rows {rows} context {args.context} a cluster of {splits} splits: {t:7.1f} us  "
                  f"{moved / t / 1e6:5.2f} TB/s")
        k.decode_attention = "balanced"
        k._splits.clear()


def prefill_attention(k, args) -> None:
    """One prompt portion of `rows` tokens whose last token is at position `context` - 1, by both prefill kernels;
    ten launches between the events, so that the host's share (two tensor maps a launch) is hidden."""
    heads, kv_heads, d, page = 32, 8, 128, 64
    for t in args.rows:
        n = max(args.context, t)
        per = -(-n // page)
        kv = torch.randn(per + 1, 2, kv_heads, page, d, device=k.device, dtype=torch.bfloat16)
        table = (torch.arange(per, device=k.device, dtype=torch.int32) + 1).view(1, per).contiguous()
        q = torch.randn(t, heads, d, device=k.device, dtype=torch.bfloat16)
        out = torch.empty_like(q)
        dev = lambda v: torch.tensor(v, device=k.device, dtype=torch.int32)   # noqa: E731
        batch = Rows(dev([0]), dev([0, t]), dev([n]), 1, t, 0, t, n, [0, t], [n])
        flops = 4 * heads * d * (t * (n - t) + t * (t + 1) // 2)
        for name, tile in (("tcgen05", 256), ("tcgen05", 128), ("mma", None)):
            k.prefill_attention, k.prefill_tile = name, tile
            batch.plan.clear()

            def ten():
                for _ in range(10):
                    k.paged_attention(out, q, kv, table, batch, 1 / math.sqrt(d), 0)
            us = timed(ten, None, 4) / 10
            label = name + (f" tile {tile}" if tile else "")
            print(f"prefill attention {label:16s} tokens {t} keys {n}: {us:7.1f} us  {flops / us / 1e6:6.0f} TFLOP/s (causal)")
        k.prefill_tile = None
    print("tcgen05 status", k.tcgen05_status())


def gemm(k, args) -> None:
    """A layer's products at each of `--rows`: the library, both tcgen05 kernels and, up to its row limit, the
    weight-streaming kernel of decode steps. Below 512 rows the product is bound by reading the weight, so the L2 is
    replaced by reading 256 MB before every run, and the weight's bytes over the time are printed as well."""
    flush_buffer = torch.zeros(256 << 20, device=k.device, dtype=torch.uint8)
    for m in args.rows:
        flush, runs = (flush_buffer, 6) if m < 512 else (None, 20)
        for name in args.shapes:
            n, kk = SHAPES[name]
            x = torch.randn(m, kk, device=k.device, dtype=torch.bfloat16)
            w = torch.randn(n, kk, device=k.device, dtype=torch.bfloat16) * 0.02
            out = torch.empty(m, n, device=k.device, dtype=torch.bfloat16)
            flops = 2 * m * n * kk
            rate = (lambda t: f"{flops / t / 1e6:5.0f} TFLOP/s") if flush is None else (lambda t: f"{2 * n * kk / t / 1e6:5.2f} TB/s")
            t_lib = timed(lambda: torch.mm(x, w.t(), out=out), flush, runs)
            t_own = timed(lambda: k.linear_tcgen05(out, x, w, pair=False), flush, runs)
            t_pair = timed(lambda: k.linear_tcgen05(out, x, w, pair=True), flush, runs)
            line = (f"{name:8s} rows {m}: cuBLAS {t_lib:7.1f} us ({rate(t_lib)})  tcgen05 {t_own:7.1f} us "
                    f"({rate(t_own)})  tcgen05 CTA pairs {t_pair:7.1f} us ({rate(t_pair)})")
            if m <= k.SKINNY_ROWS:
                t_skinny = timed(lambda: k.linear(out, x, w), flush, runs)
                line += f"  weight-streaming {t_skinny:7.1f} us ({rate(t_skinny)})"
            if m <= k.MID_ROWS:
                for split in (args.splits or [0]):
                    t_mid = timed(lambda: k.linear_mid(out, x, w, split=split), flush, runs)
                    line += f"  clustered split-k{f' ({split})' if split else ''} {t_mid:7.1f} us ({rate(t_mid)})"
            if name == "gate_up":
                act = torch.empty(m, n // 2, device=k.device, dtype=torch.bfloat16)
                t_fused = timed(lambda: k.linear_tcgen05(act, x, w, swiglu=True, pair=False), flush, runs)
                t_fused_pair = timed(lambda: k.linear_tcgen05(act, x, w, swiglu=True, pair=True), flush, runs)
                t_act = timed(lambda: k.silu_mul(act, out), flush, runs)
                line += (f"  with SwiGLU {t_fused:7.1f} us, by pairs {t_fused_pair:7.1f} us; activation kernel alone {t_act:5.1f} us")
                if m <= k.SKINNY_ROWS:
                    t_sw = timed(lambda: k.swiglu_gate_up(act, x, w), flush, runs)
                    line += f"; weight-streaming with SwiGLU {t_sw:7.1f} us"
                if m <= k.MID_ROWS:
                    t_sw = timed(lambda: k.linear_mid(act, x, w, swiglu=True), flush, runs)
                    line += f"; clustered split-k with SwiGLU {t_sw:7.1f} us"
            print(line)
    print("tcgen05 status", k.tcgen05_status())


def layer_table(k, cfg: dict, batch: int, context: int, prefill_tokens: int, hbm_gbs: float, bf16_tflops: float) -> dict:
    """Every kernel of one layer (and the head) alone, with CUDA events, at the sizes of `cfg` (config.json keys):
    a decode step of `batch` rows that hold `context` tokens, where a kernel's measure is the bytes it must read
    (weights once, the rows' cache) over its time against the copy bandwidth `hbm_gbs`; and a prompt of
    `prefill_tokens` tokens, where it is flops over time against `bf16_tflops`. The L2 is replaced before every run of
    a decode kernel. {"decode": {kernel: {"us", "mb", "gbs", "frac"}}, "prefill": {kernel: {"us", "gflop", "tflops",
    "frac"}}}; the decode products run as the engine runs them (norm, rotation, cache write, SwiGLU and the residual
    sum folded in where the kernel table folds them)."""
    from ..parts.base import Scaled
    h, d, hq, hkv, inter, vocab = (cfg[x] for x in ("hidden_size", "head_dim", "num_attention_heads", "num_key_value_heads",
                                                    "intermediate_size", "vocab_size"))
    eps, page, dev, bf = float(cfg["rms_norm_eps"]), 64, k.device, torch.bfloat16
    flush = torch.zeros(256 << 20, device=dev, dtype=torch.uint8)
    g = torch.Generator(device=dev).manual_seed(1)
    rand = lambda *shape, scale=1.0: (torch.randn(*shape, device=dev, generator=g) * scale).to(bf)   # noqa: E731
    w_qkv, w_o = rand((hq + 2 * hkv) * d, h, scale=0.02), rand(h, hq * d, scale=0.02)
    w_gu, w_down, w_head = rand(2 * inter, h, scale=0.02), rand(h, inter, scale=0.02), rand(vocab, h, scale=0.02)
    gain_h, gain_d = torch.ones(h, device=dev, dtype=bf), torch.ones(d, device=dev, dtype=bf)
    positions_max = max(context, prefill_tokens) + 1
    inv = 1.0 / (float(cfg["rope_theta"]) ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    angle = torch.arange(positions_max, dtype=torch.float32)[:, None] * inv[None, :]
    table = torch.cat((angle.cos(), angle.sin()), dim=-1).contiguous().to(dev)
    i32 = lambda v: torch.tensor(v, device=dev, dtype=torch.int32)   # noqa: E731

    def rows_of(n_rows: int, tokens_each: int, kv_each: int):
        per = -(-kv_each // page)
        kv = rand(n_rows * per + 1, 2, hkv, page, d)
        block = torch.arange(n_rows * per, device=dev, dtype=torch.int32).view(n_rows, per).contiguous()
        starts = list(range(0, n_rows * tokens_each + 1, tokens_each))
        rows = Rows(i32(list(range(n_rows))), i32(starts), i32([kv_each] * n_rows), n_rows, n_rows * tokens_each,
                    n_rows if tokens_each == 1 else 0, tokens_each, kv_each, starts, [kv_each] * n_rows)
        pos = torch.cat([torch.arange(kv_each - tokens_each, kv_each, dtype=torch.int32) for _ in range(n_rows)]).to(dev)
        write = torch.cat([block[r].repeat_interleave(page)[kv_each - tokens_each:kv_each] * page
                           + (torch.arange(kv_each - tokens_each, kv_each, device=dev, dtype=torch.int32) % page)
                           for r in range(n_rows)]).to(torch.int32).contiguous()
        return kv, block, rows, pos.contiguous(), write

    out: dict = {"decode": {}, "prefill": {}}

    # ---- one decode layer: `batch` rows of one token
    m = batch
    kv, block, rows, pos, write = rows_of(m, 1, context)
    stream = torch.randn(m, h, device=dev, generator=g)
    x = rand(m, h)
    ss = torch.full((-(-h // 16), 16), float(h) / (-(-h // 16) * 16), device=dev)       # sums of squares of unit rows
    q, o = torch.empty(m, hq, d, device=dev, dtype=bf), torch.empty(m, hq, d, device=dev, dtype=bf)
    act, logits = torch.empty(m, inter, device=dev, dtype=bf), torch.empty(m, vocab, device=dev, dtype=torch.float32)
    scaled = Scaled(x, ss, eps, h) if m <= k.SKINNY_ROWS else x
    scale = 1 / math.sqrt(d)

    def first_product():
        if not k.qkv_rope(q, scaled, w_qkv, pos, table, d, gain_d, gain_d, eps, 0.0, kv, write, hq, hkv, d):
            qkv = torch.empty(m, w_qkv.shape[0], device=dev, dtype=bf)
            k.linear(qkv, x, w_qkv)
            k.qk_norm_rope_kv_write(q, qkv, pos, table, d, gain_d, gain_d, eps, 0.0, kv, write, hq, hkv, d)

    def closing(x_in, w):
        if k.linear_link(stream, x_in, w, gain_h, eps, 0.0) is None:
            y = torch.empty(m, w.shape[0], device=dev, dtype=bf)
            k.linear(y, x_in, w)
            k.add_rmsnorm(torch.empty(m, h, device=dev, dtype=bf), stream, y, gain_h, eps, 0.0, None)

    decode = (("qkv+norm+rope+write", first_product, w_qkv.numel() * 2),
              ("attention", lambda: k.paged_attention(o, q, kv, block, rows, scale, 0), m * context * hkv * d * 4),
              ("o_proj+add+norm", lambda: closing(o.view(m, hq * d), w_o), w_o.numel() * 2),
              ("gate_up+swiglu", lambda: k.swiglu_gate_up(act, scaled, w_gu), w_gu.numel() * 2),
              ("down+add+norm", lambda: closing(act, w_down), w_down.numel() * 2),
              ("lm_head", lambda: k.linear(logits, x, w_head), w_head.numel() * 2))
    for name, fn, moved in decode:
        us = timed(fn, flush)
        out["decode"][name] = {"us": round(us, 1), "mb": round(moved / 1e6, 1), "gbs": round(moved / us / 1e3, 0),
                               "frac": round(moved / us / 1e3 / hbm_gbs, 3)}
    del kv, block, rows

    # ---- one prefill layer: one prompt of `prefill_tokens` tokens
    t = prefill_tokens
    kv, block, rows, pos, write = rows_of(1, t, t)
    stream = torch.randn(t, h, device=dev, generator=g)
    x, delta = rand(t, h), rand(t, h)
    qkv = torch.empty(t, w_qkv.shape[0], device=dev, dtype=bf)
    q, o = torch.empty(t, hq, d, device=dev, dtype=bf), torch.empty(t, hq, d, device=dev, dtype=bf)
    act, y, normed = torch.empty(t, inter, device=dev, dtype=bf), torch.empty(t, h, device=dev, dtype=bf), torch.empty(t, h, device=dev, dtype=bf)
    prefill = (("add+norm", lambda: k.add_rmsnorm(normed, stream, delta, gain_h, eps, 0.0, None), 0),
               ("qkv", lambda: k.linear(qkv, x, w_qkv), 2 * t * w_qkv.numel()),
               ("norm+rope+write", lambda: k.qk_norm_rope_kv_write(q, qkv, pos, table, d, gain_d, gain_d, eps, 0.0, kv, write, hq, hkv, d), 0),
               ("attention", lambda: k.paged_attention(o, q, kv, block, rows, scale, 0), 4 * hq * d * t * (t + 1) // 2),
               ("o_proj", lambda: k.linear(y, o.view(t, hq * d), w_o), 2 * t * w_o.numel()),
               ("gate_up+swiglu", lambda: k.swiglu_gate_up(act, x, w_gu), 2 * t * w_gu.numel()),
               ("down", lambda: k.linear(y, act, w_down), 2 * t * w_down.numel()))
    for name, fn, flops in prefill:
        def ten(fn=fn):
            for _ in range(10):
                fn()
        us = timed(ten, None, 4) / 10
        out["prefill"][name] = {"us": round(us, 1), "gflop": round(flops / 1e9, 1), "tflops": round(flops / us / 1e6, 0),
                                "frac": round(flops / us / 1e6 / bf16_tflops, 3)}
    return out


def chain(k, args) -> None:
    """A decode layer's four products on `--rows` rows (o_proj + residual + norm, gate/up + SwiGLU, down + residual +
    norm, next QKV) as launches of their own and as phases of one persistent kernel; the L2 replaced before each."""
    h, d, hq, hkv, inter = 4096, 128, 32, 8, 12288
    flush = torch.zeros(256 << 20, device=k.device, dtype=torch.uint8)
    bf = torch.bfloat16
    rand = lambda *shape: (torch.randn(*shape, device=k.device) * 0.02).to(bf)   # noqa: E731
    w_o, w_gu, w_down, w_qkv = rand(h, hq * d), rand(2 * inter, h), rand(h, inter), rand((hq + 2 * hkv) * d, h)
    gain = torch.ones(h, device=k.device, dtype=bf)
    moved = 2 * (w_o.numel() + w_gu.numel() + w_down.numel() + w_qkv.numel())
    for m in args.rows:
        o = torch.randn(m, hq * d, device=k.device).to(bf)
        stream = torch.randn(m, h, device=k.device)
        act, qkv = torch.empty(m, inter, device=k.device, dtype=bf), torch.empty(m, w_qkv.shape[0], device=k.device, dtype=bf)

        def layer():
            rows = k.linear_link(stream, o, w_o, gain, 1e-6, 0.0)
            k.swiglu_gate_up(act, rows, w_gu)
            rows2 = k.linear_link(stream, act, w_down, gain, 1e-6, 0.0)
            k.linear(qkv, rows2, w_qkv)
            k.flush()
        for chained, label in (("", "four launches"), ("tickets", "one launch, a ticket a tile"), ("ring", "one persistent kernel, a ring")):
            k.chain = chained
            t = timed(layer, flush)
            print(f"four products, rows {m}, {label:36s}: {t:7.1f} us  {moved / t / 1e6:5.2f} TB/s")
        singles = (("o_proj+add+norm", lambda: k.linear_link(stream, o, w_o, gain, 1e-6, 0.0), w_o),
                   ("down+add+norm", lambda: k.linear_link(stream, act, w_down, gain, 1e-6, 0.0), w_down))
        for name, fn, w in singles:
            for chained in ("", "tickets", "ring"):
                k.chain = chained

                def one(fn=fn):
                    fn()
                    k.flush()
                t = timed(one, flush)
                print(f"  {name:16s} rows {m} {(chained + ', alone') if chained else 'its own kernel':18s}: {t:6.1f} us  {2 * w.numel() / t / 1e6:5.2f} TB/s")
        k.chain = ""
    print("status", k.tcgen05_status())


def in_graph(calls, reps: int = 12) -> float:
    """Microseconds a call of `calls` takes on average when `reps` rounds of them run back to back in a CUDA graph
    (the fastest of five replays)."""
    for fn in calls:
        fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(reps):
            for fn in calls:
                fn()
    graph.replay()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(5):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        end.record()
        torch.cuda.synchronize()
        best = min(best, start.elapsed_time(end) * 1e3 / (reps * len(calls)))
    return best


def layer(k, args) -> None:
    """The kernels of one decode layer at Qwen3-8B sizes, each back to back in a graph: the four products plain, and
    as the engine runs them (the attention's first with q/k norm, rotation and cache write; the mixer's and the
    feed-forward's last with the residual sum and the next norm; SwiGLU's on rows that lack their norm's scale), and
    the attention over `--context` keys. The bytes a kernel must read over the copy bandwidth stand beside each time."""
    from ..parts.base import Scaled
    heads, kvh, d, hidden, inter, page = 32, 8, 128, 4096, 12288, 64
    dev, bf = k.device, torch.bfloat16
    rand = lambda *shape: torch.randn(*shape, device=dev, dtype=bf) * 0.02   # noqa: E731
    inv = 1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    angle = torch.arange(args.context + 1, dtype=torch.float32)[:, None] * inv[None, :]
    table = torch.cat((angle.cos(), angle.sin()), dim=-1).contiguous().to(dev)
    gain_d, gain_h = torch.ones(d, device=dev, dtype=bf), torch.ones(hidden, device=dev, dtype=bf)
    ideal = lambda numel: 2 * numel / 6.55e6                            # noqa: E731  (us at 6.55 TB/s)
    for m in args.rows:
        x, act, attn = rand(m, hidden) * 50, rand(m, inter) * 50, rand(m, heads * d) * 50
        positions = torch.randint(0, args.context, (m,), dtype=torch.int32, device=dev)
        cache = torch.zeros(64, 2, kvh, page, d, device=dev, dtype=bf)
        write = torch.randperm(64 * page)[:m].to(torch.int32).to(dev)
        q = torch.empty(m, heads, d, device=dev, dtype=bf)
        h = torch.randn(m, hidden, device=dev)
        unscaled = Scaled(x, torch.rand(hidden // 16, 16, device=dev), 1e-6, hidden) if m <= k.SKINNY_ROWS else None
        shapes = {"qkv": ((heads + 2 * kvh) * d, hidden), "o": (hidden, heads * d), "gate_up": (2 * inter, hidden), "down": (hidden, inter)}
        for name, (n, kk) in shapes.items():
            ws = [rand(n, kk) for _ in range(4 if n * kk < 60e6 else 2)]
            src = {"qkv": x, "o": attn, "gate_up": x, "down": act}[name]
            out = torch.empty(m, n // 2 if name == "gate_up" else n, device=dev, dtype=bf)
            if name == "gate_up":
                plain = in_graph([(lambda w=w: k.swiglu_gate_up(out, src, w)) for w in ws])
                fused = in_graph([(lambda w=w: k.swiglu_gate_up(out, unscaled, w)) for w in ws]) if unscaled else None
                what = "with SwiGLU", "the same on rows that lack their norm's scale"
            elif name == "qkv":
                plain = in_graph([(lambda w=w: k.linear(out, src, w)) for w in ws])
                rope = lambda rows, w: k.qkv_rope(q, rows, w, positions, table, d, gain_d, gain_d, 1e-6, 0.0, cache, write, heads, kvh, d)   # noqa: E731
                fused = in_graph([(lambda w=w: rope(src, w)) for w in ws]) if rope(src, ws[0]) else None
                what = "plain", "with q/k norm, rotation and cache write"
                if fused is not None and unscaled is not None:
                    late = in_graph([(lambda w=w: rope(unscaled, w)) for w in ws])
                    what = what[0], what[1] + f" (on rows that lack their norm's scale {late:6.2f} us)"
            else:
                plain = in_graph([(lambda w=w: k.linear(out, src, w)) for w in ws])
                fused = in_graph([(lambda w=w: k.linear_link(h, src, w, gain_h, 1e-6, 0.0)) for w in ws]) \
                    if k.linear_link(h, src, ws[0], gain_h, 1e-6, 0.0) is not None else None
                what = "plain", "with the residual sum and the next norm"
            line = f"rows {m:3d} {name:8s} {what[0]}: {plain:6.2f} us"
            if fused is not None:
                line += f"; {what[1]}: {fused:6.2f} us"
            print(line + f"  (the weight at the copy bandwidth: {ideal(n * kk):5.1f} us)")
            del ws
        per = -(-args.context // page)
        caches = [torch.randn(m * per + 1, 2, kvh, page, d, device=dev, dtype=bf) for _ in range(max(2, min(8, int(400e6 // (m * per * page * kvh * d * 4)) + 1)))]
        blocks = torch.arange(m * per, device=dev, dtype=torch.int32).view(m, per).contiguous()
        ar = torch.arange(m + 1, device=dev, dtype=torch.int32)
        batch = Rows(ar[:m].contiguous(), ar, torch.full((m,), args.context, device=dev, dtype=torch.int32), m, m, m, 1, args.context)
        o = torch.empty_like(q)
        t = in_graph([(lambda c=c: k.paged_attention(o, q, c, blocks, batch, 1 / math.sqrt(d), 0)) for c in caches])
        print(f"rows {m:3d} attention over {args.context} keys: {t:6.2f} us  (its cache at the copy bandwidth: {ideal(m * args.context * kvh * d * 2):5.1f} us)")
        del caches
    print("status", k.tcgen05_status())


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("what", choices=("decode_attention", "gemm", "prefill_attention", "chain", "layer"))
    ap.add_argument("--rows", type=int, nargs="*", default=None)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--splits", type=int, nargs="*", default=None)
    ap.add_argument("--cluster", type=int, nargs="*", default=None, help="decode attention: cluster sizes to time")
    ap.add_argument("--shapes", nargs="*", default=list(SHAPES), choices=list(SHAPES))
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args()
    k = load_kernels(args.device)
    with torch.inference_mode():
        if args.what == "decode_attention":
            args.rows = args.rows or [8, 64, 1]
            decode_attention(k, args)
        elif args.what == "chain":
            args.rows = args.rows or [1, 8, 16]
            chain(k, args)
        elif args.what == "layer":
            args.rows = args.rows or [8, 1, 16, 64]
            layer(k, args)
        elif args.what == "prefill_attention":
            args.rows = args.rows or [2048]
            prefill_attention(k, args)
        else:
            args.rows = args.rows or [2048]
            gemm(k, args)


if __name__ == "__main__":
    main()
