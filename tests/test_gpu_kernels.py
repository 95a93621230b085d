"""Each CUDA kernel alone against its plain torch twin (tests/ref_kernels.py), at sizes other than the engine's
tests use: widths and vocabularies that are no power of two, head sizes in steps of 16, odd groups, ragged rows,
page edges, windows. Where random inputs would average a fault away, one key is made to dominate."""
from __future__ import annotations

import ctypes
import math
import types

import pytest
import torch

import plain_qwen3 as plain
from holon_b200.engine.batch import Rows
from holon_b200.kernels.cuda import KernelError
from ref_kernels import RefKernels

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
REF = RefKernels()


@pytest.fixture(scope="module")
def K():
    from holon_b200.kernels import load_kernels
    return load_kernels(DEV)


def rand(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def close(got, want, dtype, scale=1.0):
    tol = (2e-5 if dtype == torch.float32 else 1.6e-2) * scale
    diff = (got.float().cpu() - want.float()).abs().max().item()
    assert diff <= tol, f"difference {diff} > {tol}"


@pytest.mark.parametrize("hidden", [96, 100, 4096, 5128, 10])       # (multiples of 8 take 16 bytes a load, the others 2)
def test_embed(K, hidden):
    for dtype in DTYPES:
        table = rand(389, hidden, dtype=dtype)
        ids = torch.tensor([0, 388, 5, 5, 77], dtype=torch.int32)
        out, want = torch.full((5, hidden), float("nan"), device=DEV), torch.empty(5, hidden)
        K.embed(out, table.to(DEV), ids.to(DEV))
        REF.embed(want, table, ids)
        assert torch.equal(out.cpu(), want)


@pytest.mark.parametrize("dim", [96, 1000, 4096, 13000])
@pytest.mark.parametrize("dtype", DTYPES)
def test_add_rmsnorm(K, dim, dtype):
    h, delta, w = rand(7, dim, seed=1), rand(7, dim, dtype=dtype, seed=2), (1 + rand(dim, seed=3) * 0.1)
    for wdt in {dtype, torch.float32}:                   # a norm weight stored in 32 bits stays 32-bit
        for index in (None, torch.tensor([6, 0, 3], dtype=torch.int32)):
            for d in (delta, None):
                hg, hw = h.clone().to(DEV), h.clone()
                rows = 7 if index is None else 3
                out, want = torch.empty(rows, dim, dtype=dtype, device=DEV), torch.empty(rows, dim, dtype=dtype)
                K.add_rmsnorm(out, hg, d.to(DEV) if d is not None else None, w.to(wdt).to(DEV), 1e-5, 0.0,
                              index.to(DEV) if index is not None else None)
                REF.add_rmsnorm(want, hw, d, w.to(wdt), 1e-5, 0.0, index)
                close(out, want, dtype, scale=4)
                assert torch.allclose(hg.cpu(), hw, atol=1e-6)       # the stream holds the sum (or is untouched)
    x = rand(5, dim, dtype=dtype, seed=4)
    out, want = torch.empty_like(x, device=DEV), torch.empty_like(x)
    K.rmsnorm(out, x.to(DEV), w.to(dtype).to(DEV), 1e-6, 1.0)
    REF.rmsnorm(want, x, w.to(dtype), 1e-6, 1.0)
    close(out, want, dtype, scale=8)


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(K, dtype):
    gu = rand(9, 2 * 176, dtype=dtype, scale=3.0)
    out, want = torch.empty(9, 176, dtype=dtype, device=DEV), torch.empty(9, 176, dtype=dtype)
    K.silu_mul(out, gu.to(DEV))
    REF.silu_mul(want, gu)
    close(out, want, dtype, scale=8)


@pytest.mark.parametrize("m,n,k", [(1, 389, 96), (5, 64, 7), (70, 130, 33), (129, 257, 1024), (3, 1000, 4098)])
def test_gemm_f32(K, m, n, k):
    x, w = rand(m, k, seed=1), rand(n, k, seed=2)
    out = torch.empty(m, n, device=DEV)
    K.linear(out, x.to(DEV), w.to(DEV))
    want = (x.double() @ w.double().T).float()
    assert (out.cpu() - want).abs().max().item() <= 3e-6 * math.sqrt(k) * 4
    # a row's result does not depend on the rows beside it
    alone = torch.empty(1, n, device=DEV)
    K.linear(alone, x[m - 1:].contiguous().to(DEV), w.to(DEV))
    assert torch.equal(alone[0], out[m - 1])


@pytest.mark.parametrize("m,n,k", [(1, 389, 96), (9, 1000, 176), (200, 96, 192)])
def test_linear_bf16(K, m, n, k):
    x, w = rand(m, k, dtype=torch.bfloat16, seed=1), rand(n, k, dtype=torch.bfloat16, seed=2)
    want = x.float() @ w.float().T
    out = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    K.linear(out, x.to(DEV), w.to(DEV))
    close(out, want, torch.bfloat16, scale=want.abs().max().item())
    logits = torch.empty(m, n, dtype=torch.float32, device=DEV)          # the head's form: 32-bit out
    K.linear(logits, x.to(DEV), w.to(DEV))
    assert (logits.cpu() - want).abs().max().item() <= 1e-3 * want.abs().max().item()


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16, 17])
@pytest.mark.parametrize("n,k", [(389, 96), (4096, 4096), (1000, 12288), (160, 104), (9500, 256)])
def test_linear_bf16_few_rows(K, m, n, k):
    """Decode-sized products take the weight-streaming kernel (up to 16 rows), others the library's."""
    x, w = rand(m, k, dtype=torch.bfloat16, seed=1), rand(n, k, dtype=torch.bfloat16, seed=2, scale=0.05)
    want = x.float() @ w.float().T
    for out_dtype in (torch.bfloat16, torch.float32):
        out = torch.full((m, n), float("nan"), dtype=out_dtype, device=DEV)
        K.linear(out, x.to(DEV), w.to(DEV))
        tol = (1.6e-2 if out_dtype == torch.bfloat16 else 2e-3) * max(1.0, want.abs().max().item())
        assert (out.float().cpu() - want).abs().max().item() <= tol


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 256, 256), (5, 40, 72), (300, 389, 96), (2048, 1024, 512),
                                   (130, 6144, 4096), (257, 4096, 12288)])
@pytest.mark.parametrize("pair", [False, True])
def test_linear_tcgen05(K, m, n, k, pair):
    """The tcgen05 / TMA / TMEM products (one CTA a tile; two CTAs a tile): whole tiles, ragged edges in every
    dimension, long k."""
    x, w = rand(m, k, dtype=torch.bfloat16, seed=1), rand(n, k, dtype=torch.bfloat16, seed=2, scale=0.05)
    want = x.float() @ w.float().T
    for out_dtype in (torch.bfloat16, torch.float32):
        out = torch.full((m, n), float("nan"), dtype=out_dtype, device=DEV)
        K.linear_tcgen05(out, x.to(DEV), w.to(DEV), pair=pair)
        assert K.tcgen05_status() == 0
        tol = (1.6e-2 if out_dtype == torch.bfloat16 else 2e-3) * max(1.0, want.abs().max().item())
        assert (out.float().cpu() - want).abs().max().item() <= tol


@pytest.mark.parametrize("m,inter,k", [(128, 128, 64), (70, 176, 96), (512, 1000, 328), (300, 12288, 4096)])
@pytest.mark.parametrize("pair", [False, True])
def test_swiglu_tcgen05(K, m, inter, k, pair):
    x, w = rand(m, k, dtype=torch.bfloat16, seed=3), rand(2 * inter, k, dtype=torch.bfloat16, seed=4, scale=0.1)
    gate_up = x.float() @ w.float().T
    want = torch.nn.functional.silu(gate_up[:, :inter]) * gate_up[:, inter:]
    out = torch.full((m, inter), float("nan"), dtype=torch.bfloat16, device=DEV)
    K.linear_tcgen05(out, x.to(DEV), w.to(DEV), swiglu=True, pair=pair)
    assert K.tcgen05_status() == 0
    assert (out.float().cpu() - want).abs().max().item() <= 2e-2 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("bn", [32, 128, 144, 176, 240])
def test_linear_tcgen05_pair_tile_widths(K, bn):
    """The CTA-pair product at tile widths other than the one it would choose (the last 32-column piece of a tile partly
    outside it, w's rows split 72 + 72 or 88 + 88 between the CTAs), and SwiGLU at its narrower widths."""
    m, n, k = 300, 1000, 328
    x, w = rand(m, k, dtype=torch.bfloat16, seed=5), rand(n, k, dtype=torch.bfloat16, seed=6, scale=0.05)
    want = x.float() @ w.float().T
    try:
        K.lib.hb_gemm_tcgen05_pair_width(bn)
        for out_dtype in (torch.bfloat16, torch.float32):
            out = torch.full((m, n), float("nan"), dtype=out_dtype, device=DEV)
            K.linear_tcgen05(out, x.to(DEV), w.to(DEV), pair=True)
            assert K.tcgen05_status() == 0
            tol = (1.6e-2 if out_dtype == torch.bfloat16 else 2e-3) * max(1.0, want.abs().max().item())
            assert (out.float().cpu() - want).abs().max().item() <= tol
        if bn % 64 == 0:
            inter = n // 2
            act = torch.nn.functional.silu(want[:, :inter]) * want[:, inter:]
            out = torch.full((m, inter), float("nan"), dtype=torch.bfloat16, device=DEV)
            K.linear_tcgen05(out, x.to(DEV), w.to(DEV), swiglu=True, pair=True)
            assert K.tcgen05_status() == 0
            assert (out.float().cpu() - act).abs().max().item() <= 2e-2 * max(1.0, act.abs().max().item())
    finally:
        K.lib.hb_gemm_tcgen05_pair_width(0)


@pytest.mark.parametrize("m", [1, 17, 40, 64])
@pytest.mark.parametrize("n,k", [(389, 96), (4096, 4096), (1000, 12288), (160, 104), (9500, 256), (256, 64)])
@pytest.mark.parametrize("split", [0, 1, 3, 8])
def test_products_of_up_to_64_rows_summed_over_a_cluster(K, m, n, k, split):
    """csrc/gemm_mid.cu alone: plain products (bfloat16 and 32-bit results) and SwiGLU's, every cluster size, sizes that
    are no multiple of the tile, of the k block or of four, and more CTAs in a cluster than k blocks."""
    x, w = rand(m, k, dtype=torch.bfloat16, seed=5), rand(n, k, dtype=torch.bfloat16, seed=6, scale=0.1)
    want = x.float() @ w.float().T
    for dtype in (torch.bfloat16, torch.float32):
        out = torch.full((m, n), float("nan"), dtype=dtype, device=DEV)
        K.linear_mid(out, x.to(DEV), w.to(DEV), split=split)
        close(out, want, dtype, scale=max(1.0, float(want.abs().max())))
    if n % 2 == 0:
        inter = n // 2
        want = torch.nn.functional.silu(want[:, :inter]) * want[:, inter:]
        out = torch.full((m, inter), float("nan"), dtype=torch.bfloat16, device=DEV)
        K.linear_mid(out, x.to(DEV), w.to(DEV), swiglu=True, split=split)
        assert (out.float().cpu() - want).abs().max().item() <= 2e-2 * max(1.0, want.abs().max().item())
    assert K.tcgen05_status() == 0


def test_products_of_up_to_64_rows_refuse_what_they_do_not_take(K):
    x, w = rand(65, 64, dtype=torch.bfloat16, seed=1).to(DEV), rand(32, 64, dtype=torch.bfloat16, seed=2).to(DEV)
    with pytest.raises(KernelError, match="65 rows"):
        K.linear_mid(torch.empty(65, 32, dtype=torch.bfloat16, device=DEV), x, w)
    with pytest.raises(KernelError, match="no multiple of 8"):
        K.linear_mid(torch.empty(4, 32, dtype=torch.bfloat16, device=DEV), x[:4, :60].contiguous(), w[:, :60].contiguous())
    with pytest.raises(KernelError, match="clusters of 9"):
        K.linear_mid(torch.empty(4, 32, dtype=torch.bfloat16, device=DEV), x[:4], w, split=9)


@pytest.mark.parametrize("m", [1, 8, 13, 16, 40])
@pytest.mark.parametrize("inter,k", [(176, 96), (12288, 4096), (1000, 328)])
def test_swiglu_gate_up(K, m, inter, k):
    x, w = rand(m, k, dtype=torch.bfloat16, seed=3), rand(2 * inter, k, dtype=torch.bfloat16, seed=4, scale=0.1)
    gate_up = x.float() @ w.float().T
    want = torch.nn.functional.silu(gate_up[:, :inter]) * gate_up[:, inter:]
    out = torch.full((m, inter), float("nan"), dtype=torch.bfloat16, device=DEV)
    K.swiglu_gate_up(out, x.to(DEV), w.to(DEV))
    assert (out.float().cpu() - want).abs().max().item() <= 2e-2 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,head_dim,rotary,page", [(6, 3, 80, 80, 8), (5, 1, 32, 16, 5), (8, 8, 128, 128, 64)])
def test_qk_norm_rope_kv_write(K, dtype, heads, kv_heads, head_dim, rotary, page):
    t, pages = 11, 6
    qkv = rand(t, (heads + 2 * kv_heads) * head_dim, dtype=dtype, seed=5)
    positions = torch.tensor([0, 1, 2, 40, 41, 7, 8, 9, 10, 11, 299], dtype=torch.int32)
    inv = 1.0 / (1e4 ** (torch.arange(0, rotary, 2, dtype=torch.float32) / rotary))
    ang = torch.arange(300, dtype=torch.float32)[:, None] * inv[None]
    table = torch.cat((ang.cos(), ang.sin()), -1).contiguous()
    qw, kw = (1 + rand(head_dim, seed=6) * 0.1).to(dtype), (1 + rand(head_dim, seed=7) * 0.1).to(dtype)
    write = torch.randperm(pages * page, generator=torch.Generator().manual_seed(8))[:t].to(torch.int32)
    write[3] = -1                                                             # a padded token writes nothing
    for weights in ((qw, kw), (None, None)):
        kv = rand(pages, 2, kv_heads, page, head_dim, dtype=dtype, seed=9)   # garbage: untouched cells must stay
        kvg, q, qg = kv.clone().to(DEV), torch.empty(t, heads, head_dim, dtype=dtype), None
        qg = torch.empty(t, heads, head_dim, dtype=dtype, device=DEV)
        g = lambda x: x.to(DEV) if x is not None else None               # noqa: E731
        K.qk_norm_rope_kv_write(qg, qkv.to(DEV), positions.to(DEV), table.to(DEV), rotary, g(weights[0]),
                                g(weights[1]), 1e-6, 0.0, kvg, write.to(DEV), heads, kv_heads, head_dim)
        REF.qk_norm_rope_kv_write(q, qkv, positions, table, rotary, weights[0], weights[1], 1e-6, 0.0, kv, write,
                                  heads, kv_heads, head_dim)
        close(qg, q, dtype, scale=8)
        close(kvg, kv, dtype, scale=8)
        v_got = kvg.cpu()[:, 1]
        assert torch.equal(v_got, kv[:, 1])                                   # values are copied bit for bit
    qg2 = torch.empty(t, heads, head_dim, dtype=dtype, device=DEV)            # a run that only reads the cache
    K.qk_norm_rope_kv_write(qg2, qkv.to(DEV), positions.to(DEV), table.to(DEV), rotary, None, None, 0.0, 0.0, None,
                            None, heads, kv_heads, head_dim)
    assert torch.equal(qg2, qg)


def paged_case(heads, kv_heads, head_dim, page, rows_spec, dtype, seed=0, window=0):
    """rows_spec: (tokens held before the step, new tokens) per row. Pages are handed out in a shuffled order."""
    g = torch.Generator().manual_seed(seed)
    need = [-(-(a + b) // page) for a, b in rows_spec]
    pages = sum(need) + 3
    order = torch.randperm(pages - 1, generator=g).tolist()
    slots = len(rows_spec) + 1
    table = torch.full((slots, max(need) + 1), pages - 1, dtype=torch.int32)
    kv = torch.randn(pages, 2, kv_heads, page, head_dim, generator=g).to(dtype)
    at = 0
    row_slot = torch.randperm(slots, generator=g)[:len(rows_spec)].to(torch.int32)
    for b, n in enumerate(need):
        table[row_slot[b], :n] = torch.tensor(order[at:at + n], dtype=torch.int32)
        at += n
    qs = torch.tensor([0] + [b for _, b in rows_spec], dtype=torch.int32).cumsum(0).to(torch.int32)
    kv_len = torch.tensor([a + b for a, b in rows_spec], dtype=torch.int32)
    t = int(qs[-1])
    q = torch.randn(t, heads, head_dim, generator=g).to(dtype)
    n_decode = 0
    while n_decode < len(rows_spec) and rows_spec[n_decode][1] == 1:
        n_decode += 1
    host = Rows(row_slot, qs, kv_len, len(rows_spec), t, n_decode, max(b for _, b in rows_spec), int(kv_len.max()))
    return q, kv, table, host


def on_device(rows):
    return Rows(rows.row_slot.to(DEV), rows.query_start.to(DEV), rows.kv_len.to(DEV), rows.n_rows, rows.n_tokens,
                rows.n_decode, rows.max_q, rows.max_kv, rows.query_start.numpy(), rows.kv_len.numpy())


# (heads, kv heads, head size, page): production's, the widest tensor-core head, odd groups and pages, a group of 20
# (two 16-row tiles in the decode kernel), and a head of 320 that bfloat16 hands to the CUDA-core kernel
GEOMETRIES = [(32, 8, 128, 64), (16, 4, 256, 16), (6, 1, 48, 4), (8, 2, 64, 16), (4, 4, 16, 7), (14, 2, 112, 32),
              (40, 2, 64, 16), (2, 1, 320, 8)]
PREFILL_ROWS = [(0, 1), (0, 17), (5, 16), (31, 33), (0, 64), (100, 7), (16, 16), (63, 2), (0, 130)]
DECODE_ROWS = [(0, 1), (15, 1), (16, 1), (99, 1), (999, 1), (2500, 1), (63, 1), (64, 1)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("geometry", GEOMETRIES)
@pytest.mark.parametrize("kind", ["prefill", "decode", "mixed"])
@pytest.mark.parametrize("window", [0, 20])
def test_paged_attention(K, dtype, geometry, kind, window):
    heads, kv_heads, head_dim, page = geometry
    spec = {"prefill": PREFILL_ROWS, "decode": DECODE_ROWS, "mixed": DECODE_ROWS[:4] + PREFILL_ROWS[:5]}[kind]
    q, kv, table, rows = paged_case(heads, kv_heads, head_dim, page, spec, dtype, seed=len(spec) + window)
    scale = 1 / math.sqrt(head_dim)
    want = torch.empty_like(q)
    REF.paged_attention(want, q, kv, table, rows, scale, window)
    out = torch.full_like(q, float("nan"), device=DEV)
    K.paged_attention(out, q.to(DEV), kv.to(DEV), table.to(DEV), on_device(rows), scale, window)
    close(out, want, dtype, scale=4)
    if dtype == torch.bfloat16 and head_dim == 128 and page % 64 == 0:      # this shape has two prefill kernels: the other one too
        before, K.prefill_attention = K.prefill_attention, "mma"
        try:
            other = torch.full_like(q, float("nan"), device=DEV)
            K.paged_attention(other, q.to(DEV), kv.to(DEV), table.to(DEV), on_device(rows), scale, window)
        finally:
            K.prefill_attention = before
        close(other, want, dtype, scale=4)
    again = torch.empty_like(out)
    K.paged_attention(again, q.to(DEV), kv.to(DEV), table.to(DEV), on_device(rows), scale, window)
    assert torch.equal(out, again)                                            # run to run identical


@pytest.mark.parametrize("geometry", [(32, 8, 128, 64), (40, 2, 64, 16), (6, 1, 48, 4), (16, 4, 256, 128)])
@pytest.mark.parametrize("window", [0, 300])
def test_decode_attention_with_keys_shared_out_evenly(K, geometry, window):
    """The decode kernel whose CTAs each take an equal stretch of all rows' 64-key tiles: rows of very different
    lengths, with CTA counts that put a stretch's ends inside rows, at rows' ends and across several short rows, with
    more CTAs than tiles, and with a group of 20 heads (two 16-head tiles per kv head); against the plain formula and
    against the kernel that cuts every row into equal parts."""
    heads, kv_heads, head_dim, page = geometry
    spec = [(2999, 1), (0, 1), (63, 1), (64, 1), (700, 1), (5, 1), (1300, 1), (127, 1), (128, 1)]
    q, kv, table, rows = paged_case(heads, kv_heads, head_dim, page, spec, torch.bfloat16, seed=17 + window)
    scale = 1 / math.sqrt(head_dim)
    want = torch.empty_like(q)
    REF.paged_attention(want, q, kv, table, rows, scale, window)
    args = (q.to(DEV), kv.to(DEV), table.to(DEV), on_device(rows), scale, window)
    before = K.decode_attention, K.decode_ctas
    try:
        K.decode_attention = "splits"
        cut = torch.full_like(q, float("nan"), device=DEV)
        K.paged_attention(cut, *args)
        close(cut, want, torch.bfloat16, scale=4)
        K.decode_attention = "balanced"
        for ctas in (None, 1, 2, 7, 50, 443, 5000):
            K.decode_ctas = ctas
            out = torch.full_like(q, float("nan"), device=DEV)
            K.paged_attention(out, *args)
            close(out, want, torch.bfloat16, scale=4)
            again = torch.full_like(q, float("nan"), device=DEV)
            K.paged_attention(again, *args)
            assert torch.equal(out, again), ctas
        K.decode_attention = "auto"
        assert K.decode_mode([8192] + [500] * 31) == "balanced" and K.decode_mode([8192] * 8) == "splits"
        assert K.decode_mode([300, 20, 5000]) == "splits" and K.decode_mode(None) == "splits"
    finally:
        K.decode_attention, K.decode_ctas = before


@pytest.mark.parametrize("heads,kv_heads,page", [(8, 2, 64), (4, 4, 128), (6, 1, 64)])
@pytest.mark.parametrize("window", [0, 100])
def test_prefill_attention_tcgen05(K, heads, kv_heads, page, window):
    """The tcgen05 prefill kernel (head size 128): ragged rows beside decode rows, portions that continue a context,
    more than one 128-query tile, long contexts that force the lagging maximum to be rescaled."""
    spec = [(300, 1), (0, 1), (0, 17), (5, 128), (31, 33), (0, 200), (1000, 130), (64, 64), (0, 700)]
    q, kv, table, rows = paged_case(heads, kv_heads, 128, page, spec, torch.bfloat16, seed=3 + window)
    q[40:60] *= 4.0                                     # peaked rows: the running maximum moves by more than the lag
    scale = 1 / math.sqrt(128)
    want = torch.empty_like(q)
    REF.paged_attention(want, q, kv, table, rows, scale, window)
    before = K.prefill_attention
    K.prefill_attention = "tcgen05"
    try:
        out = torch.full_like(q, float("nan"), device=DEV)
        K.paged_attention(out, q.to(DEV), kv.to(DEV), table.to(DEV), on_device(rows), scale, window)
        assert K.tcgen05_status() == 0
    finally:
        K.prefill_attention = before
    close(out, want, torch.bfloat16, scale=4)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("page", [16, 64])
def test_attention_finds_one_far_key(K, dtype, page):
    """One key among 700 is made to match the query; the output must be that key's value. The key sits at page edges,
    at the first and the last position, and, with a window, just inside and just outside it."""
    heads, kv_heads, head_dim, n = 8, 2, 64, 700
    scale = 1 / math.sqrt(head_dim)
    for window in (0, 128):
        for target in (0, page - 1, page, 5 * page - 1, 5 * page, n - 129, n - 128, n - 2, n - 1):
            q, kv, table, rows = paged_case(heads, kv_heads, head_dim, page, [(n - 1, 1), (n - 3, 3)], dtype, seed=target)
            kv.mul_(0.05)
            for b in range(2):
                slot = int(rows.row_slot[b])
                p, off = int(table[slot, target // page]), target % page
                for t in range(int(rows.query_start[b]), int(rows.query_start[b + 1])):
                    for h in range(heads):
                        direction = torch.nn.functional.normalize(q[t, h].float(), dim=0)
                        q[t, h] = (direction * 8).to(dtype)
                    kv[p, 0, :, off] = 0
                for hk in range(kv_heads):                        # the key matches the mean direction of its group
                    group = q[int(rows.query_start[b]), hk * 4:(hk + 1) * 4].float()
                    kv[p, 0, hk, off] = (torch.nn.functional.normalize(group.mean(0), dim=0) * 60).to(dtype)
                    kv[p, 1, hk, off] = 3.0
            want = torch.empty_like(q)
            REF.paged_attention(want, q, kv, table, rows, scale, window)
            out = torch.empty_like(q, device=DEV)
            K.paged_attention(out, q.to(DEV), kv.to(DEV), table.to(DEV), on_device(rows), scale, window)
            close(out, want, dtype, scale=4)
            visible = window == 0 or (n - 1) - target < window
            first_row = out[0].float().cpu()                      # the decode row, at position n - 1
            if visible:
                assert (first_row - 3.0).abs().max() < 0.2, (window, target)
            else:
                assert first_row.abs().max() < 1.0, (window, target)


@pytest.mark.parametrize("heads,kv_heads,head_dim,hidden", [(32, 8, 128, 4096), (6, 1, 64, 104), (4, 4, 32, 64), (20, 2, 128, 320)])
@pytest.mark.parametrize("m,wide", [(1, False), (8, False), (13, False), (17, False), (40, False), (64, False),
                                    (17, True), (32, True)])
@pytest.mark.parametrize("norm", ["bfloat16", "float32", None])
def test_qkv_product_with_norm_rotation_and_cache_write(K, heads, kv_heads, head_dim, hidden, m, norm, wide, monkeypatch):
    """The decode step's QKV product with q/k norm, rotation and cache write in its epilogue (up to 16 rows: a cluster
    of CTAs per head; 17 to 64: a cluster per 256 weight rows that shares the k range) against the product followed by
    the separate kernel: queries, and the pages that were written. `wide`: 17 to 32 rows through the mma.sync kernel
    with four tiles of x a warp (weights of a few MB) instead."""
    monkeypatch.setattr(K, "mid_mode", "0" if wide else "all")
    monkeypatch.setattr(K, "skinny32", wide)
    monkeypatch.setattr(K, "MID_WEIGHT", 1 << 40 if wide else K.MID_WEIGHT)   # (whatever the weight's size)
    g = torch.Generator().manual_seed(heads + m)
    x = (torch.randn(m, hidden, generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn((heads + 2 * kv_heads) * head_dim, hidden, generator=g) * 0.05).to(torch.bfloat16)
    wdt = {"bfloat16": torch.bfloat16, "float32": torch.float32, None: None}[norm]
    qw = (1 + 0.1 * torch.randn(head_dim, generator=g)).to(wdt) if wdt else None
    kw = (1 + 0.1 * torch.randn(head_dim, generator=g)).to(wdt) if wdt else None
    positions = torch.randint(0, 500, (m,), generator=g, dtype=torch.int32)
    inv = 1.0 / (1e4 ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    angle = torch.arange(512, dtype=torch.float32)[:, None] * inv[None, :]
    table = torch.cat((angle.cos(), angle.sin()), dim=-1).contiguous()
    pages, page = 9, 16
    write = torch.randperm(pages * page, generator=g)[:m].to(torch.int32)
    if m > 2:
        write[1] = -1                                                  # a token whose key and value go nowhere
    dev = lambda t: None if t is None else t.to(DEV)                   # noqa: E731
    outs = []
    for fused in (True, False):
        kv = torch.full((pages, 2, kv_heads, page, head_dim), 7.0, dtype=torch.bfloat16, device=DEV)
        q = torch.full((m, heads, head_dim), float("nan"), dtype=torch.bfloat16, device=DEV)
        args = (dev(positions), dev(table), head_dim, dev(qw), dev(kw), 1e-5, 0.0, kv, dev(write), heads, kv_heads, head_dim)
        if fused:
            assert K.qkv_rope(q, dev(x), dev(w), *args)
        else:
            qkv = torch.empty(m, w.shape[0], dtype=torch.bfloat16, device=DEV)
            K.linear(qkv, dev(x), dev(w))
            K.qk_norm_rope_kv_write(q, qkv, *args)
        outs.append((q.float().cpu(), kv.float().cpu()))
    (q1, kv1), (q2, kv2) = outs
    assert torch.isfinite(q1).all()
    scale = max(1.0, float(q2.abs().max()))
    assert (q1 - q2).abs().max() <= 2e-2 * scale and (kv1 - kv2).abs().max() <= 2e-2 * max(scale, float(kv2.abs().max()))
    assert ((kv1 == 7.0) == (kv2 == 7.0)).all()                        # the same places were written


@pytest.mark.parametrize("hidden,wide", [(4096, 4096), (96, 192), (200, 72), (1024, 3072)])
@pytest.mark.parametrize("m,rows32", [(1, False), (8, False), (16, False), (17, False), (32, False), (33, False),
                                      (64, False), (17, True), (32, True)])
@pytest.mark.parametrize("norm", ["bfloat16", "float32"])
def test_residual_sum_and_norm_inside_the_products_around_them(K, hidden, wide, m, norm, rows32, monkeypatch):
    """A product that adds itself into the 32-bit stream and leaves the next norm's rows unscaled, and the three
    products that take such rows (plain, SwiGLU, QKV with rotation), against the separate kernels: product,
    add_rmsnorm, product. Up to 16 rows the stream itself must come out the same to the bit (both ways sum in the
    same order); from 17 rows on the separate product is the library's, whose sums may round another way: the stream
    then agrees to one rounding of the product. (Every product its own launch here; the same products as phases of one
    kernel: test_products_chained_in_one_kernel.)"""
    monkeypatch.setattr(K, "chain", "")
    monkeypatch.setattr(K, "mid_mode", "0" if rows32 else "all")       # rows32: the mma.sync kernel with four tiles of x a warp
    monkeypatch.setattr(K, "skinny32", rows32)
    monkeypatch.setattr(K, "MID_WEIGHT", 1 << 40 if rows32 else K.MID_WEIGHT)  # (whatever the weight's size)
    g = torch.Generator().manual_seed(hidden + m)
    dev = lambda t: t.to(DEV)                                          # noqa: E731
    x = dev((torch.randn(m, wide, generator=g) * 0.5).to(torch.bfloat16))
    w = dev((torch.randn(hidden, wide, generator=g) * 0.05).to(torch.bfloat16))
    h0 = dev(torch.randn(m, hidden, generator=g) * 2.0)
    gain = dev((1 + 0.1 * torch.randn(hidden, generator=g)).to(getattr(torch, norm)))
    eps, offset = 1e-5, 0.25
    norm_part = types.SimpleNamespace(weight=types.SimpleNamespace(tensor=gain))
    assert K.can_link(m, hidden, norm_part) and not K.can_link(33 if rows32 else 65, hidden, norm_part)
    # the separate kernels
    delta = torch.empty(m, hidden, dtype=torch.bfloat16, device=DEV)
    K.linear(delta, x, w)
    h_want, xn = h0.clone(), torch.empty(m, hidden, dtype=torch.bfloat16, device=DEV)
    K.add_rmsnorm(xn, h_want, delta, gain, eps, offset, None)
    # the linked product
    h_got = h0.clone()
    rows = K.linear_link(h_got, x, w, gain, eps, offset)
    assert rows is not None and rows.shape == (m, hidden)
    if m <= 16:
        assert rows.ss.shape == (-(-hidden // 16), 16) and torch.equal(h_got, h_want) and (rows.ss[:, m:] == 0).all()
    else:
        assert rows.ss.shape == ((-(-hidden // 16), 32) if rows32 else (-(-hidden // 256), 64))
        assert (h_got - h_want).abs().max() <= 2.0 ** -7 * float(delta.float().abs().max())
    ss = rows.ss.double().sum(0)[:m].cpu()
    assert torch.allclose(ss, h_got.double().pow(2).sum(-1).cpu(), rtol=1e-5)
    # 1. a plain product of the rows
    w2 = dev((torch.randn(176, hidden, generator=g) * 0.05).to(torch.bfloat16))
    want, got = (torch.empty(m, 176, dtype=torch.bfloat16, device=DEV) for _ in range(2))
    K.linear(want, xn, w2)
    K.linear(got, rows, w2)
    close(got, want.cpu(), torch.bfloat16, scale=2 * max(1.0, float(want.abs().max())))
    # 2. SwiGLU's first product
    w3 = dev((torch.randn(2 * 208, hidden, generator=g) * 0.05).to(torch.bfloat16))
    want, got = (torch.empty(m, 208, dtype=torch.bfloat16, device=DEV) for _ in range(2))
    K.swiglu_gate_up(want, xn, w3)
    K.swiglu_gate_up(got, rows, w3)
    close(got, want.cpu(), torch.bfloat16, scale=2 * max(1.0, float(want.abs().max())))
    # 3. the attention's first product with q/k norm, rotation and cache write
    heads, kv_heads, head_dim = 4, 2, 64
    w4 = dev((torch.randn((heads + 2 * kv_heads) * head_dim, hidden, generator=g) * 0.05).to(torch.bfloat16))
    qw, kw = (dev((1 + 0.1 * torch.randn(head_dim, generator=g)).to(torch.bfloat16)) for _ in range(2))
    inv = 1.0 / (1e4 ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    angle = torch.arange(64, dtype=torch.float32)[:, None] * inv[None, :]
    table = dev(torch.cat((angle.cos(), angle.sin()), dim=-1).contiguous())
    positions = dev(torch.randint(0, 64, (m,), generator=g, dtype=torch.int32))
    write = dev(torch.randperm(80, generator=g)[:m].to(torch.int32))
    outs = []
    for source in (xn, rows):
        kv = torch.full((5, 2, kv_heads, 16, head_dim), 1024.0, dtype=torch.bfloat16, device=DEV)
        q = torch.full((m, heads, head_dim), float("nan"), dtype=torch.bfloat16, device=DEV)
        assert K.qkv_rope(q, source, w4, positions, table, head_dim, qw, kw, 1e-6, 0.0, kv, write, heads, kv_heads, head_dim)
        outs.append((q.float().cpu(), kv.float().cpu()))
    (q1, kv1), (q2, kv2) = outs
    assert torch.isfinite(q2).all() and (q1 - q2).abs().max() <= 4e-2 * max(1.0, float(q1.abs().max()))
    written = kv1 != 1024.0
    assert (written == (kv2 != 1024.0)).all() and written.sum() == 2 * m * kv_heads * head_dim
    assert (kv1 - kv2)[written].abs().max() <= 4e-2 * max(1.0, float(kv1[written].abs().max()))
    # where the kernel does not apply, nothing is done
    assert K.linear_link(h_got.double().float()[:, :hidden], x.float(), w.float(), gain, eps, offset) is None


@pytest.mark.parametrize("hidden,inter,heads,kv_heads,head_dim", [(4096, 12288, 32, 8, 128), (1024, 3072, 16, 8, 128),
                                                                  (96, 176, 6, 1, 48), (64, 128, 4, 2, 16), (200, 72, 2, 2, 24)])
@pytest.mark.parametrize("m", [1, 7, 16])
@pytest.mark.parametrize("kind", ["tickets", "ring"])
def test_products_chained_in_one_kernel(K, hidden, inter, heads, kv_heads, head_dim, m, kind, monkeypatch):
    """A decode layer's products on the same few rows (attention output -> o_proj + residual + post norm -> gate/up with
    SwiGLU -> down + residual + next input norm -> next QKV, twice over) queued and run in one launch, against the same
    products as launches of their own. "tickets": every CTA a tile of one of the products, in order, the arithmetic
    that of the separate kernels: the same bits. "ring": one persistent kernel whose CTAs take equal shares of chunks
    whatever the shapes, so tiles are summed across CTAs: sums may differ in the last bits, never more. The odd sizes
    leave CTAs without work and tiles with ragged ends."""
    from holon_b200.parts.base import Scaled
    monkeypatch.setattr(K, "mid_mode", "0")                            # (the separate launches: the mma.sync kernel's too)
    g = torch.Generator().manual_seed(hidden + 3 * m)
    dev = lambda t: t.to(DEV)                                          # noqa: E731
    mat = lambda n, k: dev((torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16))   # noqa: E731
    gain = lambda n: dev((1 + 0.1 * torch.randn(n, generator=g)).to(torch.bfloat16))     # noqa: E731
    qkv_rows = (heads + 2 * kv_heads) * head_dim
    layers = [dict(o=mat(hidden, heads * head_dim), gate_up=mat(2 * inter, hidden), down=mat(hidden, inter), qkv=mat(qkv_rows, hidden),
                   post=gain(hidden), after=gain(hidden)) for _ in range(2)]
    attn = [dev((torch.randn(m, heads * head_dim, generator=g) * 0.5).to(torch.bfloat16)) for _ in range(2)]
    h0 = dev(torch.randn(m, hidden, generator=g))
    eps = 1e-6

    def run(chain: str):
        monkeypatch.setattr(K, "chain", chain)
        h, outs, before = h0.clone(), [], (K.chain_launches, K.chain_phases)
        for layer, o in zip(layers, attn):
            rows = K.linear_link(h, o, layer["o"], layer["post"], eps, 0.0)
            act = torch.empty(m, inter, dtype=torch.bfloat16, device=DEV)
            K.swiglu_gate_up(act, rows, layer["gate_up"])
            rows2 = K.linear_link(h, act, layer["down"], layer["after"], eps, 0.0)
            qkv = torch.empty(m, qkv_rows, dtype=torch.bfloat16, device=DEV)
            K.linear(qkv, rows2, layer["qkv"])
            assert isinstance(rows, Scaled) and isinstance(rows2, Scaled)
            if chain:
                assert len(K._pending) == 4
            K.flush()                                                  # (the engine's next call, the rotation kernel, does this)
            outs.append((act.float().cpu(), qkv.float().cpu(), rows.y.float().cpu(), rows2.ss.double().sum(0).cpu()))
        counted = (K.chain_launches - before[0], K.chain_phases - before[1])
        return h.cpu(), outs, counted

    h_want, want, none = run("")
    h_got, got, counted = run(kind)
    assert none == (0, 0) and counted == (2, 8)
    if kind == "tickets":
        assert torch.equal(h_got, h_want)
        for mine, theirs in zip(got, want):
            assert all(torch.equal(a, b) for a, b in zip(mine, theirs))
    assert K.tcgen05_status() == 0
    assert torch.isfinite(h_got).all()
    # the stream: each product is rounded to bfloat16 before it is added, so a last-bit difference of a sum shows
    # either not at all or as one bfloat16 step of that product (and the second layer's products start from it)
    step = 2.0 ** -7 * (h_want - h0.cpu()).abs().max().item()
    assert (h_got - h_want).abs().max().item() <= 2 * step
    first_want, first_got = want[0][2], got[0][2]                      # the first product's rows: same inputs on both sides
    assert (first_got != first_want).float().mean().item() < 0.02
    for (act1, qkv1, y1, ss1), (act2, qkv2, y2, ss2) in zip(want, got):
        for a, b in ((act1, act2), (qkv1, qkv2), (y1, y2)):
            assert (a - b).abs().max().item() <= 1.6e-2 * max(1.0, a.abs().max().item())
        assert torch.allclose(ss1[:m], ss2[:m], rtol=1e-3)


@pytest.mark.parametrize("geometry", [(32, 8, 128, 64), (40, 2, 64, 16), (6, 1, 48, 4), (16, 4, 256, 128)])
def test_decode_attention_merged_inside_a_cluster(K, geometry):
    """2 to 16 splits of a row as a thread-block cluster that merges through distributed shared memory, rows shorter
    than the number of splits among them, against the plain formula and run to run; and the planner takes a cluster
    only while every (row, kv head) has one in the same wave."""
    heads, kv_heads, head_dim, page = geometry
    spec = [(1999, 1), (0, 1), (63, 1), (64, 1), (700, 1), (5, 1), (1300, 1), (128, 1)]
    q, kv, table, rows = paged_case(heads, kv_heads, head_dim, page, spec, torch.bfloat16, seed=31)
    scale = 1 / math.sqrt(head_dim)
    want = torch.empty_like(q)
    REF.paged_attention(want, q, kv, table, rows, scale, 0)
    args = (q.to(DEV), kv.to(DEV), table.to(DEV), on_device(rows))
    for splits in range(2, 17):
        assert K._cluster_capacity(head_dim, splits) >= 1
        outs = []
        for _ in range(2):
            out = torch.full_like(q, float("nan"), device=DEV)
            K._call("hb_attention_decode_bf16_cluster", K._p(out), K._p(args[0]), K._p(args[1]), K._i32(args[2], "table"),
                    args[2].shape[1], K._i32(args[3].row_slot, "slot"), K._i32(args[3].query_start, "start"),
                    K._i32(args[3].kv_len, "len"), len(spec), heads, kv_heads, head_dim, kv.shape[0], page,
                    ctypes.c_float(scale), 0, splits)
            outs.append(out)
        close(outs[0], want, torch.bfloat16, scale=4)
        assert torch.equal(outs[0], outs[1]), splits
    for n_rows in (1, 2, 8, 16, 64, 300):
        planned = K.decode_splits(n_rows, heads, kv_heads, 8192)
        few = K.decode_cluster_splits(n_rows, heads, kv_heads, head_dim, 8192, planned)
        pairs = n_rows * kv_heads * (-(-(heads // kv_heads) // 16))
        assert few == 0 or (2 <= few <= 16 and pairs <= K._cluster_capacity(head_dim, few)), (n_rows, few)
        if n_rows == 1 and pairs <= K._cluster_capacity(head_dim, 16):
            assert few == 16                               # one row of 128 tiles: the largest cluster, 8 tiles a CTA
        if n_rows == 300:
            assert few == 0                                # several waves: the merge kernel


@pytest.mark.parametrize("window", [0, 4096])
def test_attention_over_a_long_context(K, window):
    """20,000 keys a row at head size 128 and pages of 64 (313 pages a row, shuffled): a decode row, a two-token portion
    and a 300-token portion at the end of such contexts, through the split and the balanced decode kernels and both
    prefill kernels, against the plain formula; one far key is made to stand out in the decode row."""
    heads, kv_heads, head_dim, page, n = 8, 2, 128, 64, 20000
    spec = [(n - 1, 1), (n - 2, 2), (n - 300, 300)]
    q, kv, table, rows = paged_case(heads, kv_heads, head_dim, page, spec, torch.bfloat16, seed=23 + window)
    kv[:, 0].mul_(0.3)
    target = n - 3000 if window else 1234                             # inside the window, or far back
    slot = int(rows.row_slot[0])
    pg, off = int(table[slot, target // page]), target % page
    for hk in range(kv_heads):
        group = q[0, hk * 4:(hk + 1) * 4].float()
        kv[pg, 0, hk, off] = (torch.nn.functional.normalize(group.mean(0), dim=0) * 40).to(torch.bfloat16)
        kv[pg, 1, hk, off] = 5.0
    scale = 1 / math.sqrt(head_dim)
    want = torch.empty_like(q)
    REF.paged_attention(want, q, kv, table, rows, scale, window)
    assert (want[0].float() - 5.0).abs().max() < 0.5                  # the plain formula finds the key too
    args = (q.to(DEV), kv.to(DEV), table.to(DEV), on_device(rows), scale, window)
    before = K.decode_attention, K.prefill_attention
    try:
        for decode in ("splits", "balanced"):
            for prefill in ("tcgen05", "mma"):
                K.decode_attention, K.prefill_attention = decode, prefill
                out = torch.full_like(q, float("nan"), device=DEV)
                K.paged_attention(out, *args)
                assert K.tcgen05_status() == 0
                close(out, want, torch.bfloat16, scale=4)
    finally:
        K.decode_attention, K.prefill_attention = before


def test_sample_greedy_and_temperature(K):
    v, rows = 1531, 6
    logits = rand(rows, v, seed=3, scale=2.0)
    logits[1, 700] = logits[1, 900] = 9.0                         # equal maxima: the lowest index wins
    logits[5] = logits[2]
    params = dict(temperature=torch.tensor([0, 0, 0.7, 1.0, 1.3, 0.7]), top_k=torch.zeros(rows, dtype=torch.int32),
                  top_p=torch.ones(rows), min_p=torch.zeros(rows), seed_lo=torch.tensor([1, 2, 3, 4, 5, 3], dtype=torch.int32),
                  seed_hi=torch.tensor([0, 0, 9, 0, 1, 9], dtype=torch.int32),
                  position=torch.tensor([5, 6, 7, 8, 9, 7], dtype=torch.int32))
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    g = {k: t.to(DEV) for k, t in params.items()}
    K.sample(out, logits.to(DEV), g["temperature"], g["top_k"], g["top_p"], g["min_p"], g["seed_lo"], g["seed_hi"],
             g["position"], False)
    got = out.cpu().tolist()
    assert got[0] == int(logits[0].argmax()) and got[1] == 700
    for r in range(2, rows):
        seed = int(params["seed_lo"][r]) | (int(params["seed_hi"][r]) << 32)
        want = plain.sample(logits[r], float(params["temperature"][r]), seed, int(params["position"][r]))
        assert got[r] == want
    assert got[2] == got[5]                                        # same seed, position and logits: same token


@pytest.mark.parametrize("vocab,k", [(1531, 5), (151936, 20), (37, 37), (600, 0)])
def test_logprobs_of_the_raw_logits(K, vocab, k):
    """The chosen token's log-probability and the ranked top-k against log_softmax in float64; equal logits rank by
    ascending id, and a row with fewer finite entries than k fills the rest with id -1 and -inf."""
    rows = 5
    logits = rand(rows, vocab, seed=5 + k, scale=3.0)
    logits[1, 3] = logits[1, vocab - 1] = logits[1, 17] = 50.0          # three equal maxima
    if vocab == 37:
        logits[2, 5:] = float("-inf")                                 # five finite entries
    tokens = torch.tensor([0, vocab - 1, 3, vocab // 2, 7], dtype=torch.int32)
    chosen = torch.empty(rows, dtype=torch.float32, device=DEV)
    top_ids = torch.full((rows, k), -7, dtype=torch.int32, device=DEV)
    top = torch.full((rows, k), float("nan"), dtype=torch.float32, device=DEV)
    K.logprobs(chosen, top_ids, top, logits.to(DEV), tokens.to(DEV))
    for r in range(rows):
        own, ids, values = plain.logprobs(logits[r], int(tokens[r]), k)
        assert abs(float(chosen[r]) - own) < 2e-5 * max(1.0, abs(own)), (r, float(chosen[r]), own)
        finite = [i for i, v in zip(ids, values) if v != float("-inf")]
        got = top_ids[r].cpu().tolist()
        assert got[:len(finite)] == finite and all(i == -1 for i in got[len(finite):]), (r, got, ids)
        for a, b in zip(top[r].cpu().tolist(), values):
            assert (a == b == float("-inf")) or abs(a - b) < 2e-5 * max(1.0, abs(b))
    if k >= 3:
        assert top_ids[1, :3].cpu().tolist() == [3, 17, vocab - 1]


def test_sample_follows_the_distribution(K):
    """4096 draws of one row at positions 0..4095, against the plain implementation's float64 distribution, with and
    without filters: total variation small, filtered-out tokens never drawn."""
    v, n = 389, 4096
    row = rand(1, v, seed=11, scale=2.5)
    logits = row.expand(n, v).contiguous().to(DEV)
    for temperature, top_k, top_p, min_p in ((0.8, 0, 1.0, 0.0), (1.0, 12, 1.0, 0.0), (1.0, 0, 0.8, 0.0),
                                             (1.2, 0, 1.0, 0.05), (0.9, 40, 0.9, 0.02)):
        filtered = bool(top_k or top_p < 1 or min_p > 0)
        out = torch.empty(n, dtype=torch.int32, device=DEV)
        full = lambda x, dt: torch.full((n,), x, dtype=dt, device=DEV)   # noqa: E731
        K.sample(out, logits, full(temperature, torch.float32), full(top_k, torch.int32), full(top_p, torch.float32),
                 full(min_p, torch.float32), full(1234, torch.int32), full(0, torch.int32),
                 torch.arange(n, dtype=torch.int32, device=DEV), filtered)
        probs = plain.distribution(row[0], temperature, top_k, top_p, min_p)
        counts = torch.bincount(out.cpu().long(), minlength=v).double() / n
        assert counts[probs == 0].sum() == 0
        assert 0.5 * (counts - probs).abs().sum() < 0.12
        for i in range(0, n, 97):                                  # and token by token
            assert int(out[i]) == plain.draw(probs, plain.uniform(1234, i))
