"""The decode attention entry point that allocates nothing (`hb_attention_decode_bf16_static`), called through its
exported C symbol, against the entry point that takes scratch from the caller.

Some users of the library cannot allocate when they call it: a server that gave all free device memory to its cache
at start, or a program in another language that sees only the C symbols. For them the library carries its own scratch
array. This test makes two calls in a row with different inputs and different splits (the array keeps the first
call's contents, which must not leak into the second: each result must equal the other entry point's bit for bit, and
the plain attention within the kernel tests' bound), and checks that a launch too large for the array is refused
with a message instead of run. The file sorts last on purpose: a run that stops at the first failure has then already
run every other test.
"""
from __future__ import annotations

import ctypes
import math
import types

import pytest
import torch

from ref_kernels import RefKernels

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def case(seed, rows, heads, kv_heads, head_dim, page, lengths):
    g = torch.Generator().manual_seed(seed)
    need = [-(-n // page) for n in lengths]
    pages = sum(need) + 2
    order = torch.randperm(pages, generator=g).tolist()
    table = torch.zeros(rows, max(need), dtype=torch.int32)
    at = 0
    for b, n in enumerate(need):
        table[b, :n] = torch.tensor(order[at:at + n], dtype=torch.int32)
        at += n
    t = lambda x: x.to(DEV).contiguous()                        # noqa: E731
    return dict(q=t(torch.randn(rows, heads, head_dim, generator=g).bfloat16()),
                kv=t(torch.randn(pages, 2, kv_heads, page, head_dim, generator=g).bfloat16()), table=t(table),
                row_slot=t(torch.arange(rows, dtype=torch.int32)), query_start=t(torch.arange(rows + 1, dtype=torch.int32)),
                kv_len=t(torch.tensor(lengths, dtype=torch.int32)), rows=rows, heads=heads, kv_heads=kv_heads,
                head_dim=head_dim, pages=pages, page=page)


def test_static_scratch_entry_point_matches_the_one_that_takes_scratch():
    from holon_b200.kernels.build import library_path
    lib = ctypes.CDLL(str(library_path()))
    lib.hb_last_error.restype = ctypes.c_char_p
    lib.hb_attention_decode_static_capacity.restype = ctypes.c_size_t
    lib.hb_attention_decode_scratch_floats.restype = ctypes.c_size_t
    capacity = lib.hb_attention_decode_static_capacity()
    assert capacity == 2 * 1024 * 1024
    stream = ctypes.c_void_p(torch.cuda.current_stream(torch.device(DEV)).cuda_stream)
    p = lambda x: ctypes.c_void_p(x.data_ptr())                 # noqa: E731

    def both(c, splits, window):
        common = (p(c["q"]), p(c["kv"]), p(c["table"]), c["table"].shape[1], p(c["row_slot"]), p(c["query_start"]),
                  p(c["kv_len"]), c["rows"], c["heads"], c["kv_heads"], c["head_dim"], c["pages"], c["page"],
                  ctypes.c_float(1 / math.sqrt(c["head_dim"])), window, splits, stream)
        floats = lib.hb_attention_decode_scratch_floats(c["rows"], c["heads"], c["head_dim"], splits)
        assert 0 < floats <= capacity
        scratch = torch.empty(floats, dtype=torch.float32, device=DEV)
        want = torch.full_like(c["q"], float("nan"))
        assert lib.hb_attention_decode_bf16(p(want), p(scratch), *common) == 0, lib.hb_last_error()
        got = torch.full_like(c["q"], float("nan"))
        assert lib.hb_attention_decode_bf16_static(p(got), *common) == 0, lib.hb_last_error()
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got, want)            # the same launch with other scratch, a fixed-order merge: bit for bit
        rows = types.SimpleNamespace(query_start=c["query_start"].cpu(), row_slot=c["row_slot"].cpu(),
                                     kv_len=c["kv_len"].cpu(), n_rows=c["rows"])
        plain = torch.empty(c["q"].shape, dtype=torch.float32)
        RefKernels().paged_attention(plain, c["q"].float().cpu(), c["kv"].float().cpu(), c["table"].cpu(), rows,
                                     1 / math.sqrt(c["head_dim"]), window)
        assert (got.float().cpu() - plain).abs().max().item() <= 1.6e-2 * 4      # the kernel tests' bfloat16 bound
        return got

    first = both(case(1, 5, 8, 2, 128, 16, [700, 64, 1, 333, 1500]), splits=5, window=0)
    second = both(case(2, 3, 12, 4, 64, 64, [90, 2049, 640]), splits=7, window=100)      # other sizes, stale scratch
    assert first.shape == (5, 8, 128) and second.shape == (3, 12, 64)

    big = case(3, 64, 32, 8, 128, 64, [70] * 64)
    out = torch.empty_like(big["q"])
    rc = lib.hb_attention_decode_bf16_static(
        p(out), p(big["q"]), p(big["kv"]), p(big["table"]), big["table"].shape[1], p(big["row_slot"]),
        p(big["query_start"]), p(big["kv_len"]), 64, 32, 8, 128, big["pages"], 64, ctypes.c_float(0.1), 0, 16, stream)
    assert rc == 1                                               # refused, nothing launched
    message = lib.hb_last_error().decode()
    assert "4259840" in message and str(capacity) in message
