"""Tiny configurations and small tools shared by the tests."""
from __future__ import annotations

import json

import torch
from safetensors.torch import save_file

from holon_b200.weights import RandomSource

# Two tiny Qwen3 configurations that differ in every size and option: head counts and groups (2 and 6), head sizes
# (16 and 48, the second no power of two and heads × head size ≠ hidden), width, layers, vocabulary (256 and 389,
# the second odd), eps, rotation base, tied or own head.
TINY_A = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, intermediate_size=128, vocab_size=256, rope_theta=10000.0,
              rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=128)
TINY_B = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=3, hidden_size=96, num_attention_heads=6,
              num_key_value_heads=1, head_dim=48, intermediate_size=176, vocab_size=389, rope_theta=1000000.0,
              rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=512)
# The second tiny configuration of the benchmark's own list (head size 32, intermediate 160, vocabulary 384): all
# powers of two or multiples of 32 where TINY_B is not, one KV head for six query heads.
TINY_C = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=3, hidden_size=96, num_attention_heads=6,
              num_key_value_heads=1, head_dim=32, intermediate_size=160, vocab_size=384, rope_theta=1000000.0,
              rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=512)
TINY = {"a": (TINY_A, 0), "b": (TINY_B, 1), "c": (TINY_C, 1)}


def make_folder(tmp_path, name: str, sharpen: float = 2.0, dtype=torch.bfloat16):
    """A model folder of tiny configuration `name` with seeded random weights. `sharpen` scales the q- and k-norm
    weights: with unit gains the scores of random weights stay near zero and attention is close to an average over
    all keys, which hides a wrong mask or a wrong page; scaled gains make single keys stand out."""
    config, seed = TINY[name]
    folder = tmp_path / f"tiny_{name}"
    folder.mkdir(parents=True, exist_ok=True)
    tensors = {}
    for stored, t in RandomSource(config, seed, dtype=dtype).tensors():
        if stored.endswith(("q_norm.weight", "k_norm.weight")):
            t = (t.float() * sharpen).to(dtype)
        tensors[stored] = t.contiguous()
    (folder / "config.json").write_text(json.dumps(config))
    save_file(tensors, str(folder / "model.safetensors"))
    return folder


def random_prompt(vocab: int, n: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


# ---------------------------------------------------------------- what the reference's own engine produced (tests/golden)

def golden_engine():
    """tests/golden/qwen3_tiny_engine.json: the reference sampler's uniforms and draws, and the tokens its engine
    generated on the CPU for the two tiny models of tests/golden/make_golden.py."""
    import pathlib
    return json.loads((pathlib.Path(__file__).resolve().parent / "golden" / "qwen3_tiny_engine.json").read_text())


def golden_folder(tmp_path, name: str, golden: dict):
    """A model folder holding the very weights the golden tokens of model `name` were generated with (float32), or a
    skip if this torch's random generator draws other weights than the recording one did."""
    import importlib.util
    import pathlib

    import pytest
    path = pathlib.Path(__file__).resolve().parent / "golden" / "make_golden.py"
    spec = importlib.util.spec_from_file_location("make_golden", path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    config = module.CONFIGS[name]
    weights = module.tiny_weights(config, module.SEEDS[name])
    recorded = golden["engine"][name]["checksum"]
    if abs(module.checksum(weights) - recorded) > 1e-9 * recorded:
        pytest.skip("this torch draws other random weights than the one that recorded the golden tokens")
    folder = tmp_path / f"golden_{name}"
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config))
    save_file({k: v.contiguous() for k, v in weights.items()}, str(folder / "model.safetensors"))
    return folder, config, weights
