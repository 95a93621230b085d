"""Weights: names, merged rows, precisions, the one error that lists every fault, the random-weights folder."""
from __future__ import annotations

import json

import pytest
import torch
from safetensors.torch import save_file

from helpers import TINY_A, TINY_B
from holon_b200.config import resolve_architecture
from holon_b200.parts import BuildContext, Model
from holon_b200.weights import (NameMap, RandomSource, SafetensorsSource, WeightError, load_weights,
                                write_model_folder)


def model_of(raw, dtype=torch.float32):
    arch = resolve_architecture(raw)
    spec = arch.recipe(arch.parse(raw))
    return Model(spec, BuildContext("cpu", dtype, None, max_positions=16)), spec


def test_names_map_both_ways():
    _, spec = model_of(TINY_A)
    names = NameMap(spec.weight_rules)
    assert names.ours("model.layers.12.self_attn.q_norm.weight") == "layers.12.mixer.q_norm.weight"
    assert names.stored("layers.3.ffn.down_proj.weight") == "model.layers.3.mlp.down_proj.weight"
    assert names.ours("model.embed_tokens.weight") == "embed.weight" and names.ours("lm_head.weight") == "head.weight"
    assert names.ours("model.layers.x.mlp.up_proj.weight") is None and names.ours("model.norm.weight.extra") is None


def test_random_folder_round_trip(tmp_path):
    for raw, seed in ((TINY_A, 0), (TINY_B, 1)):
        folder = write_model_folder(RandomSource(raw, seed), tmp_path / f"m{seed}")
        assert json.loads((folder / "config.json").read_text()) == raw and (folder / "model.safetensors").is_file()
        source = SafetensorsSource(folder)
        stored = dict(source.tensors())
        assert all(t.dtype == torch.bfloat16 for t in stored.values())
        assert ("lm_head.weight" in stored) == (not raw["tie_word_embeddings"])
        again = dict(RandomSource(raw, seed).tensors())
        assert all(torch.equal(stored[k], again[k]) for k in stored)                # seeded: the same tensors again
        other = dict(RandomSource(raw, seed + 1).tensors())
        assert not torch.equal(stored["model.norm.weight"], other["model.norm.weight"])
        gains = stored["model.layers.0.self_attn.q_norm.weight"].float()
        assert abs(float(gains.mean()) - 1) < 0.2 and float(stored["model.embed_tokens.weight"].float().std()) < 0.03
        model, spec = model_of(raw)
        held = load_weights(model, spec, source.tensors(), torch.float32, "cpu")
        assert held == sum(p.tensor.numel() * 4 for _, p in model.params())
        h, d = raw["num_attention_heads"], raw["head_dim"]
        qkv = model.layers[0].mixer.qkv.weight.tensor                               # q, k, v rows stacked in one weight
        assert torch.equal(qkv[:h * d], stored["model.layers.0.self_attn.q_proj.weight"].float())
        assert torch.equal(qkv[h * d:h * d + raw["num_key_value_heads"] * d],
                           stored["model.layers.0.self_attn.k_proj.weight"].float())
        gu = model.layers[1].ffn.gate_up.weight.tensor
        assert torch.equal(gu[raw["intermediate_size"]:], stored["model.layers.1.mlp.up_proj.weight"].float())


def test_precisions(tmp_path):
    """bfloat16 engine: matrices and tables in bfloat16; a norm weight stored in 32 bits stays 32-bit."""
    tensors = {k: (t.float() if k.endswith("norm.weight") and "layers.0" in k else t)
               for k, t in RandomSource(TINY_A, 0).tensors()}
    model, spec = model_of(TINY_A, torch.bfloat16)
    load_weights(model, spec, tensors.items(), torch.bfloat16, "cpu")
    dtypes = {name: p.tensor.dtype for name, p in model.params()}
    assert dtypes["layers.0.input_norm.weight"] == torch.float32 == dtypes["layers.0.mixer.q_norm.weight"]
    assert dtypes["layers.1.input_norm.weight"] == torch.bfloat16
    assert dtypes["layers.0.mixer.qkv.weight"] == torch.bfloat16 == dtypes["embed.weight"]
    model32, _ = model_of(TINY_A)
    load_weights(model32, spec, tensors.items(), torch.float32, "cpu")
    assert {p.tensor.dtype for _, p in model32.params()} == {torch.float32}


def test_one_error_lists_every_fault():
    tensors = dict(RandomSource(TINY_B, 1).tensors())
    del tensors["model.layers.1.mlp.up_proj.weight"], tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    tensors["model.layers.7.mlp.up_proj.weight"] = torch.zeros(2, 2)                 # a layer the model does not have
    tensors["model.layers.2.self_attn.k_proj.weight"] = torch.zeros(5, 96)
    model, spec = model_of(TINY_B)
    with pytest.raises(WeightError) as e:
        load_weights(model, spec, tensors.items(), torch.float32, "cpu")
    err = e.value
    assert sorted(err.missing) == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert sorted(err.unexpected) == ["model.layers.0.self_attn.rotary_emb.inv_freq", "model.layers.7.mlp.up_proj.weight"]
    assert [(n, tuple(g), w) for n, g, w in err.shapes] == [("model.layers.2.self_attn.k_proj.weight", (5, 96), (48, 96))]
    text = str(err)
    for piece in ("missing (2)", "unexpected (2)", "wrong shape", "(5, 96)", "(48, 96)"):
        assert piece in text


def test_tied_head_ignores_a_stored_copy_and_folder_errors(tmp_path):
    tensors = dict(RandomSource(TINY_A, 0).tensors())
    tensors["lm_head.weight"] = torch.zeros(256, 64)
    model, spec = model_of(TINY_A)
    load_weights(model, spec, tensors.items(), torch.float32, "cpu")                 # no error: the copy is skipped
    assert model.head.weight is None
    with pytest.raises(FileNotFoundError, match="config.json"):
        SafetensorsSource(tmp_path)
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    with pytest.raises(FileNotFoundError, match="safetensors"):
        SafetensorsSource(tmp_path)
    save_file({"a": torch.zeros(1)}, str(tmp_path / "m1.safetensors"))
    save_file({"a": torch.zeros(1)}, str(tmp_path / "m2.safetensors"))
    with pytest.raises(ValueError, match="both"):
        list(SafetensorsSource(tmp_path).tensors())
