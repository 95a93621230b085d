"""The plain implementation against what mxinO/holon's own CPU model computed (tests/golden/), and against itself."""
from __future__ import annotations

import importlib.util
import pathlib

import pytest
import torch
from safetensors import safe_open

import plain_qwen3 as plain

GOLDEN = pathlib.Path(__file__).resolve().parent / "golden"
_spec = importlib.util.spec_from_file_location("make_golden", GOLDEN / "make_golden.py")
make_golden = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(make_golden)


@pytest.mark.parametrize("name", ["a", "b"])
def test_plain_matches_holon_cpu_model(name):
    config = make_golden.CONFIGS[name]
    weights = make_golden.tiny_weights(config, make_golden.SEEDS[name])
    with safe_open(str(GOLDEN / "qwen3_tiny.safetensors"), framework="pt") as f:
        golden, checksum = f.get_tensor(f"{name}.logits"), float(f.get_tensor(f"{name}.checksum")[0])
    if abs(make_golden.checksum(weights) - checksum) > 1e-9 * checksum:
        pytest.skip("this torch draws other random weights than the one that recorded the golden logits")
    ours = torch.cat([plain.forward(config, weights, ids) for ids in make_golden.prompts(name)])
    assert ours.shape == golden.shape
    assert (ours - golden).abs().max().item() < 2e-6
    assert torch.equal(ours.argmax(-1), golden.argmax(-1))


def test_window_hides_old_keys():
    g = torch.Generator().manual_seed(3)
    q, k, v = (torch.randn(9, 2, 16, generator=g) for _ in range(3))
    full, win = plain.causal_attention(q, k, v), plain.causal_attention(q, k, v, window=4)
    assert torch.allclose(full[:4], win[:4])              # the first W queries see everything
    assert not torch.allclose(full[4:], win[4:])
    tail = plain.causal_attention(q[5:], k[5:], v[5:])     # the last query sees keys 5..8 only
    assert torch.allclose(win[8], tail[3], atol=1e-6)


def test_uniform_is_a_function_of_seed_and_position():
    assert plain.uniform(7, 11) == plain.uniform(7, 11)
    for seed in (0, 1, 2**40 + 5):
        us = [plain.uniform(seed, p) for p in range(200)]
        assert len(set(us)) == len(us) and all(0 < u < 1 for u in us)
        assert abs(sum(us) / len(us) - 0.5) < 0.1
    assert plain.uniform(5, 3) != plain.uniform(2**32 + 5, 3)      # the high half of the seed counts


def test_distribution_filters():
    logits = torch.tensor([2.0, 1.0, 0.5, -1.0, 3.0])
    assert plain.distribution(logits, 0.0).tolist() == [0, 0, 0, 0, 1]
    p = plain.distribution(logits, 1.0, top_k=2)
    assert (p > 0).tolist() == [True, False, False, False, True] and abs(float(p.sum()) - 1) < 1e-12
    p = plain.distribution(logits, 1.0, top_p=0.5)         # the most likely token alone already reaches 0.5
    assert (p > 0).tolist() == [False, False, False, False, True]
    p = plain.distribution(logits, 1.0, min_p=0.2)
    assert (p > 0).tolist() == [True, False, False, False, True]
    assert plain.draw(torch.tensor([0.0, 0.5, 0.0, 0.5]), 0.25) == 1
    assert plain.draw(torch.tensor([0.0, 0.5, 0.0, 0.5]), 0.75) == 3


# ---------------------------------------------------------------- sampling and generation against the reference's own

def test_uniform_and_draws_match_the_reference_sampler():
    """`plain.uniform` and `plain.sample` against the values the reference's sampler produced (tests/golden/
    make_engine_golden.py): the hash of (seed, position) for seeds on both sides of 2^32, and the inverse-CDF draw at
    two temperatures. The plain kernel table's sampler is held to the same draws."""
    import sys
    from helpers import golden_engine
    sys.path.insert(0, str(GOLDEN))
    import make_engine_golden as recorded
    from ref_kernels import RefKernels
    golden = golden_engine()
    table = iter(golden["uniform"])
    for seed in golden["seeds"]:
        for position in golden["positions"]:
            assert abs(plain.uniform(seed, position) - next(table)) < 1e-12, (seed, position)
    logits = recorded.draw_logits()
    rows = logits.shape[0]
    kernels = RefKernels()
    for case in golden["draws"]:
        t, seed, position = case["temperature"], case["seed"], case["position"]
        assert [plain.sample(row, t, seed, position) for row in logits] == case["tokens"], case
        tokens = torch.zeros(rows, dtype=torch.int32)
        full = lambda v, dt: torch.full((rows,), v, dtype=dt)                   # noqa: E731
        as_i32 = lambda v: torch.tensor([v], dtype=torch.int64).to(torch.int32).repeat(rows)   # noqa: E731
        kernels.sample(tokens, logits, full(t, torch.float32), full(0, torch.int32), full(1.0, torch.float32),
                       full(0.0, torch.float32), as_i32(seed & 0xFFFFFFFF), as_i32(seed >> 32), full(position, torch.int32), False)
        assert tokens.tolist() == case["tokens"], case


@pytest.mark.parametrize("name", ["a", "b"])
def test_plain_generation_matches_the_reference_engine(name, tmp_path):
    """Whole forward passes and `plain.sample`, token by token, against what the reference's engine generated with its
    paged cache, prompt portions beside decoding requests and seeded temperature sampling."""
    from helpers import golden_engine, golden_folder
    golden = golden_engine()
    _, config, weights = golden_folder(tmp_path, name, golden)
    work = golden["engine"][name]
    for prompt, seed, want in zip(work["prompts"], work["workload"]["seeds"], work["tokens"]):
        got = plain.generate(config, weights, prompt, work["workload"]["max_tokens"], work["workload"]["temperature"], seed)
        assert got == want
