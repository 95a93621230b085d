"""The engine at Qwen3-8B's layer sizes (hidden 4096, 32 query and 8 KV heads of 128, intermediate 12288, vocabulary
151,936, rotation base 1e6), cut to two layers so that the plain implementation can follow on the CPU: a prompt in
one step, the rest in portions and token by token, in true 32-bit and in bfloat16. The tiny configurations cannot show
a fault that needs a long reduction, a wide head or the production tile shapes; this one can."""
from __future__ import annotations

import pytest
import torch

import plain_qwen3 as plain
from helpers import random_prompt
from holon_b200.engine import StepEntry, build
from holon_b200.weights import RandomSource

pytestmark = pytest.mark.gpu

CONFIG = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=4096, num_attention_heads=32,
              num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=151936, rope_theta=1000000.0,
              rms_norm_eps=1e-6, tie_word_embeddings=False)


class Held:
    """A weight source that draws the random tensors once and hands the same ones to the engine and to the plain code."""

    def __init__(self, config, seed):
        self._config = config
        self.kept = {name: t for name, t in RandomSource(config, seed).tensors()}

    def config(self):
        return self._config

    def eos_token_ids(self):
        return ()

    def tensors(self):
        return iter(self.kept.items())


@pytest.fixture(scope="module")
def case():
    source = Held(CONFIG, seed=2)
    ids = random_prompt(CONFIG["vocab_size"], 150, 9)
    weights = {k: v.float() for k, v in source.kept.items()}
    exact = plain.forward(CONFIG, weights, ids)
    with plain.rounding(torch.bfloat16):
        rounded = plain.forward(CONFIG, weights, ids)
    del weights
    return source, ids, exact, rounded


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_portions_and_decoding_at_real_sizes(case, dtype):
    source, ids, exact, rounded = case
    b = build(source, dtype=dtype, device="cuda:0", page_size=64, max_seqs=4, max_model_len=256, max_step_tokens=256,
              pages=8)
    slot, at, rows = b.cache.admit(), 0, []
    for n in [97, 17, 2, 20] + [1] * 14:                      # a long portion, ragged ones, then token by token
        assert b.cache.reserve(slot, at + n)
        rows.append(b.runner.step([StepEntry(slot, ids[at:at + n], at, range(n))]).float().cpu())
        at += n
    assert at == len(ids)
    got = torch.cat(rows)
    diff = (got - exact).abs()
    if dtype == "float32":
        assert diff.max() <= 1e-4, float(diff.max())
        assert torch.equal(got.argmax(-1), exact.argmax(-1))
    else:
        floor = (rounded - exact).abs()
        assert diff.max() <= 2.0 * floor.max(), (float(diff.max()), float(floor.max()))
        assert diff.mean() <= 1.5 * floor.mean(), (float(diff.mean()), float(floor.mean()))
    b.cache.release(slot)
    b.cache.check()


@pytest.fixture(scope="module")
def mixed_case():
    source = Held(CONFIG, seed=2)
    prompts = {rid: random_prompt(CONFIG["vocab_size"], n, 20 + i) for i, (rid, n) in
               enumerate((("a", 268), ("b", 207), ("c", 40), ("d", 60)))}
    weights = {k: v.float() for k, v in source.kept.items()}
    want = {}
    for rid, ids in prompts.items():
        exact = plain.forward(CONFIG, weights, ids)
        with plain.rounding(torch.bfloat16):
            want[rid] = (exact, plain.forward(CONFIG, weights, ids))
    del weights
    return source, prompts, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_steps_at_real_sizes(mixed_case, dtype):
    """Up to four live requests at the production layer sizes, decode rows beside prompt portions in one step, on pages
    of 64 in a pool of eleven, so that the last request runs in a page another one gave back. The steps are cut to
    meet the kernels' own borders: a portion of 260 tokens (more than the 256 queries of the largest attention tile),
    one of 200 beside a decode row (more than the 192 rows from which SwiGLU's product runs on CTA pairs), steps of
    16 and of 17 tokens in all (the row limit of the weight-streaming products), and portions of two tokens."""
    from replay_tools import compare
    source, p, want = mixed_case
    b = build(source, dtype=dtype, device="cuda:0", page_size=64, max_seqs=4, max_model_len=320, max_step_tokens=320,
              pages=11)
    trace = [
        ([("a", 260)], []),
        ([("a", 1), ("b", 200)], []),
        ([("a", 1), ("b", 1), ("c", 14)], []),                       # 16 tokens in all
        ([("a", 1), ("b", 1), ("c", 15)], []),                       # 17
        ([("a", 1), ("b", 1), ("c", 11)], ["c"]),
        ([("a", 1), ("b", 1), ("d", 2)], []),                        # d takes the page c gave back
        ([("a", 1), ("b", 1), ("d", 30)], []),
        ([("a", 1), ("b", 1), ("d", 28)], ["d"]),
        ([("a", 1), ("b", 1)], ["a", "b"]),
    ]
    slots, at, got = {}, {rid: 0 for rid in p}, {}
    pages_of_c = None
    for step, end in trace:
        entries = []
        for rid, n in step:
            if rid not in slots:
                slots[rid] = b.cache.admit()
            assert b.cache.reserve(slots[rid], at[rid] + n)
            entries.append(StepEntry(slots[rid], p[rid][at[rid]:at[rid] + n], at[rid], range(n)))
        logits = b.runner.step(entries).float().cpu()
        k = 0
        for rid, n in step:
            for _ in range(n):
                got[(rid, at[rid])] = logits[k]
                at[rid], k = at[rid] + 1, k + 1
        group = b.cache.groups[0]
        if "c" in end:
            pages_of_c = set(group.table[slots["c"], :1].tolist())
        if ("d", 2) in step:
            assert set(group.table[slots["d"], :1].tolist()) == pages_of_c
        for rid in end:
            b.cache.release(slots.pop(rid))
        b.cache.check()
    assert at == {rid: len(ids) for rid, ids in p.items()} and not b.cache.live
    compare(got, want, dtype)
    assert b.ctx.kernels.tcgen05_status() == 0


@pytest.fixture(scope="module")
def rows_case():
    source = Held(CONFIG, seed=2)
    prompts = {f"r{i}": random_prompt(CONFIG["vocab_size"], 70, 60 + i) for i in range(4)}
    weights = {k: v.float() for k, v in source.kept.items()}
    want = {}
    for rid, ids in prompts.items():
        exact = plain.forward(CONFIG, weights, ids)
        with plain.rounding(torch.bfloat16):
            want[rid] = (exact, plain.forward(CONFIG, weights, ids))
    del weights
    return source, prompts, want


def test_steps_on_both_sides_of_every_row_limit_at_real_sizes(rows_case):
    """The products change kernels with the number of rows a step brings (up to 8 and up to 16: the mma.sync kernel with
    one and two tiles of x; SwiGLU's on the clustered tcgen05 kernel up to 64, the attention's first from 9 to 16; from
    17 the library, from 65 for every product): steps of 65, 64, 33, 32, 17, 16, 9 and 8 tokens at the production layer
    sizes, decode rows beside prompt portions, against the plain implementation."""
    from replay_tools import compare
    source, p, want = rows_case
    b = build(source, dtype="bfloat16", device="cuda:0", page_size=64, max_seqs=4, max_model_len=128, max_step_tokens=128,
              pages=9)
    trace = [[("r0", 65)], [("r1", 64)], [("r0", 1), ("r2", 32)], [("r0", 1), ("r1", 1), ("r3", 30)],
             [("r0", 1), ("r1", 1), ("r2", 15)], [("r0", 1), ("r1", 1), ("r3", 14)], [("r0", 1), ("r1", 1), ("r2", 7)],
             [("r1", 1), ("r2", 7)], [("r1", 1), ("r2", 9), ("r3", 26)]]
    assert [sum(n for _, n in step) for step in trace] == [65, 64, 33, 32, 17, 16, 9, 8, 36]
    kernels = b.ctx.kernels
    before = kernels.mid_launches
    slots, at, got = {}, {rid: 0 for rid in p}, {}
    for step in trace:
        entries = []
        for rid, n in step:
            if rid not in slots:
                slots[rid] = b.cache.admit()
            assert b.cache.reserve(slots[rid], at[rid] + n)
            entries.append(StepEntry(slots[rid], p[rid][at[rid]:at[rid] + n], at[rid], range(n)))
        logits = b.runner.step(entries).float().cpu()
        k = 0
        for rid, n in step:
            for _ in range(n):
                got[(rid, at[rid])] = logits[k]
                at[rid], k = at[rid] + 1, k + 1
    assert at == {rid: 70 for rid in p}
    assert kernels.mid_launches - before >= 2 * 8          # (SwiGLU's product of the eight steps of up to 64 rows, two layers)
    compare(got, want, "bfloat16")
    assert kernels.tcgen05_status() == 0
