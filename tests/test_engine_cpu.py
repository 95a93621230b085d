"""The engine's host side on the CPU: the step function, the cache and the scheduler driven with the plain torch
kernel table of tests/ref_kernels.py in place of the CUDA kernels, against the plain implementation."""
from __future__ import annotations

import pytest
import torch

import plain_qwen3 as plain
from helpers import TINY, make_folder, random_prompt
from holon_b200.engine import Engine, EngineConfig, SamplingParams, StepEntry, StepError, build
from holon_b200.weights import SafetensorsSource
from ref_kernels import RefKernels


def built(folder, **kw):
    args = dict(dtype="float32", device="cpu", kernels=RefKernels(), page_size=4, max_seqs=4, max_model_len=128,
                max_step_tokens=64, pages=40)
    args.update(kw)
    return build(SafetensorsSource(folder), **args)


@pytest.mark.parametrize("name", ["a", "b"])
def test_whole_prompt_and_portions_match_plain(tmp_path, name):
    folder = make_folder(tmp_path, name)
    config, weights = plain.read_folder(folder)
    ids = random_prompt(config["vocab_size"], 37, 5)
    want = plain.forward(config, weights, ids)
    b = built(folder)
    slot = b.cache.admit()
    assert b.cache.reserve(slot, len(ids))
    got = b.runner.step([StepEntry(slot, ids, 0, range(len(ids)))])
    assert (got - want).abs().max() < 1e-4
    b.cache.release(slot)
    slot, at, parts = b.cache.admit(), 0, []
    for n in (5, 2, 9, 1, 1, 13, 6):
        assert b.cache.reserve(slot, at + n)
        parts.append(b.runner.step([StepEntry(slot, ids[at:at + n], at, range(n))]))
        at += n
    assert at == len(ids)
    assert (torch.cat(parts) - want).abs().max() < 1e-4
    b.cache.check()


def test_step_refuses_bad_batches(tmp_path):
    b = built(make_folder(tmp_path, "a"))
    slot = b.cache.admit()
    with pytest.raises(StepError, match="not reserved"):
        b.runner.step([StepEntry(slot, [1, 2, 3], 0)])
    b.cache.reserve(slot, 3)
    with pytest.raises(StepError, match="start at 2"):
        b.runner.step([StepEntry(slot, [1], 2)])
    with pytest.raises(StepError, match="outside the vocabulary"):
        b.runner.step([StepEntry(slot, [1, 999, 3], 0)])
    with pytest.raises(StepError, match="not admitted"):
        b.runner.step([StepEntry(3, [1], 0)])
    assert b.runner.step([StepEntry(slot, [1, 2, 3], 0)]) is None          # nothing wanted: no logits


@pytest.mark.parametrize("name,temperature", [("a", 0.0), ("b", 0.0), ("b", 0.7)])
def test_generate_matches_plain(tmp_path, name, temperature):
    folder = make_folder(tmp_path, name)
    config, weights = plain.read_folder(folder)
    prompts = [random_prompt(config["vocab_size"], n, 20 + n) for n in (5, 17, 31, 1)]
    engine = Engine(EngineConfig(model=str(folder), device="cpu", dtype="float32", page_size=4, max_seqs=3,
                                 max_model_len=64, max_step_tokens=16, chunk_with_decode=8, state_memory=1 << 20),
                    kernels=RefKernels())
    params = [SamplingParams(temperature=temperature, max_tokens=8, seed=11 + i) for i in range(len(prompts))]
    got = engine.generate(prompts, params)
    for p, g, sp in zip(prompts, got, params):
        assert g == plain.generate(config, weights, p, 8, temperature, sp.seed)
    engine.built.cache.check()
    assert not engine.built.cache.live and engine.stats()["mixed_steps"] > 0
