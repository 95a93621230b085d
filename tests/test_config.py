"""Configuration: the typed Qwen3 configuration read from config.json keys, the architecture registry, the recipe,
the engine settings."""
from __future__ import annotations

import pytest

from helpers import TINY_A, TINY_B
from holon_b200.config import (ConfigError, EngineConfig, ModelSpec, PartRef, Run, register_architecture,
                               resolve_architecture, unregister_architecture)
from holon_b200.models.qwen3 import Qwen3Config, recipe


def test_every_size_comes_from_config_json():
    for raw in (TINY_A, TINY_B):
        cfg = Qwen3Config.from_dict(raw)
        spec = recipe(cfg)
        assert (spec.hidden, spec.vocab, len(spec.layers)) == (raw["hidden_size"], raw["vocab_size"], raw["num_hidden_layers"])
        mixer = spec.layers[0].mixer.kwargs()
        assert (mixer["heads"], mixer["kv_heads"], mixer["head_dim"]) == (
            raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"])
        assert mixer["position"].kwargs() == {"theta": raw["rope_theta"], "rotary_dim": raw["head_dim"]}
        assert mixer["qk_norm"].kwargs() == {"eps": raw["rms_norm_eps"]} == spec.norm.kwargs()
        assert spec.layers[0].ffn.kwargs() == {"inter": raw["intermediate_size"]}
        assert spec.head.kwargs() == {"tied": raw["tie_word_embeddings"]}
        assert spec.order == tuple(Run(i, i, True) for i in range(raw["num_hidden_layers"]))
        assert spec.ignore_stored == (("lm_head.",) if raw["tie_word_embeddings"] else ())


def test_missing_and_wrong_keys_are_named():
    for key in ("hidden_size", "head_dim", "rms_norm_eps", "rope_theta", "num_key_value_heads"):
        raw = {k: v for k, v in TINY_A.items() if k != key}
        with pytest.raises(ConfigError, match=key):
            Qwen3Config.from_dict(raw)
    with pytest.raises(ConfigError, match="hidden_size"):
        Qwen3Config.from_dict(dict(TINY_A, hidden_size="64"))
    with pytest.raises(ConfigError, match="multiple"):
        Qwen3Config.from_dict(dict(TINY_A, num_attention_heads=5))
    assert Qwen3Config.from_dict(dict(TINY_A, rope_theta=10000)).rope_theta == 10000.0       # an int base is fine


def test_rope_parameters_style_and_refused_options():
    raw = {k: v for k, v in TINY_A.items() if k != "rope_theta"}
    raw["rope_parameters"] = {"rope_theta": 5e5, "rope_type": "default"}
    assert Qwen3Config.from_dict(raw).rope_theta == 5e5
    with pytest.raises(NotImplementedError, match="yarn"):
        Qwen3Config.from_dict(dict(TINY_A, rope_scaling={"type": "yarn", "factor": 4}))
    for key in ("attention_bias", "use_sliding_window"):
        with pytest.raises(NotImplementedError, match=key):
            Qwen3Config.from_dict(dict(TINY_A, **{key: True}))
    assert Qwen3Config.from_dict(dict(TINY_A, use_sliding_window=False, sliding_window=4096)) is not None
    assert Qwen3Config.from_dict(dict(TINY_A, eos_token_id=[3, 9])).eos_token_ids == (3, 9)
    assert Qwen3Config.from_dict(dict(TINY_A, eos_token_id=7)).eos_token_ids == (7,)


def test_registry():
    arch = resolve_architecture(TINY_A)
    assert arch.name == "Qwen3ForCausalLM" and arch.parse(TINY_A) == Qwen3Config.from_dict(TINY_A)
    with pytest.raises(ConfigError, match="LlamaForCausalLM.*Qwen3ForCausalLM"):
        resolve_architecture({"architectures": ["LlamaForCausalLM"]})
    with pytest.raises(ConfigError, match="architectures"):
        resolve_architecture({})
    with pytest.raises(ValueError, match="registered already"):
        register_architecture("Qwen3ForCausalLM", Qwen3Config.from_dict, recipe)
    register_architecture("ToyArch", dict, lambda c: None)
    try:
        assert resolve_architecture({"architectures": ["ToyArch"]}).name == "ToyArch"
    finally:
        unregister_architecture("ToyArch")


def test_run_order_is_checked():
    ref = PartRef.of("norm", "rmsnorm", eps=1e-6)
    layer = recipe(Qwen3Config.from_dict(TINY_A)).layers[0]
    base = dict(hidden=64, vocab=256, layers=(layer, layer), embed=ref, norm=ref, head=ref, weight_rules=())
    ModelSpec(order=(Run(0, 0), Run(1, 0, fills=False), Run(1, 1), Run(0, 2)), **base)   # a layer twice; a shared entry
    with pytest.raises(ValueError, match="filled by two runs"):
        ModelSpec(order=(Run(0, 0), Run(1, 0)), **base)
    with pytest.raises(ValueError, match="before any run fills it"):
        ModelSpec(order=(Run(0, 1, fills=False), Run(1, 1)), **base)
    with pytest.raises(ValueError, match="names layer 2"):
        ModelSpec(order=(Run(2, 0),), **base)


def test_engine_config():
    with pytest.raises(ValueError, match="page_size"):
        EngineConfig(model="x", page_size=0)
    with pytest.raises(ValueError, match="dtype"):
        EngineConfig(model="x", dtype="float16")
    with pytest.raises(ValueError, match="max_seqs \\+ chunk_with_decode"):
        EngineConfig(model="x", max_seqs=64, max_step_tokens=100, chunk_with_decode=64)
    cfg = EngineConfig(model="x")
    assert (cfg.dtype, cfg.page_size, cfg.max_seqs, cfg.max_model_len, cfg.max_step_tokens, cfg.chunk_with_decode) == (
        "bfloat16", 64, 64, 8192, 4096, 0)
