"""Qwen3 dense decoder: its typed configuration and its recipe.

Grouped-query attention with a per-head RMSNorm on q and k before the rotation, a head size that config.json
gives on its own, SwiGLU, pre-norm RMSNorm blocks, full causal attention, an optionally tied head. The keys read,
the ones refused and the stored tensor names are the reference's
(plugins/holon_plugins/models/qwen3/recipe.py:10-18, 32-59).
"""
from __future__ import annotations

import dataclasses
from collections.abc import Mapping
from typing import Any

from ..config.registry import ConfigError, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartRef, Run, WeightRule


def _need(c: Mapping[str, Any], key: str, kind):
    if key not in c:
        raise ConfigError(f"config.json: missing key {key!r}")
    value = c[key]
    if kind is float and isinstance(value, int) and not isinstance(value, bool):
        value = float(value)
    if not isinstance(value, kind) or isinstance(value, bool) and kind is not bool:
        raise ConfigError(f"config.json: {key!r} must be {kind.__name__}, not {value!r}")
    return value


@dataclasses.dataclass(frozen=True)
class Qwen3Config:
    hidden_size: int
    vocab_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool = False
    max_position_embeddings: int | None = None
    eos_token_ids: tuple[int, ...] = ()

    @staticmethod
    def from_dict(c: Mapping[str, Any]) -> "Qwen3Config":
        refused = {k: c[k] for k in ("attention_bias", "use_sliding_window") if c.get(k)}
        if refused:
            raise NotImplementedError(f"qwen3: config options not supported: {refused}")
        rope = c.get("rope_parameters") or {"rope_theta": _need(c, "rope_theta", float), **(c.get("rope_scaling") or {})}
        kind = rope.get("rope_type", rope.get("type", "default"))
        if kind != "default":
            raise NotImplementedError(f"qwen3: rope type {kind!r} not supported")
        eos = c.get("eos_token_id", ())
        eos = (eos,) if isinstance(eos, int) else tuple(eos or ())
        cfg = Qwen3Config(
            hidden_size=_need(c, "hidden_size", int), vocab_size=_need(c, "vocab_size", int),
            num_hidden_layers=_need(c, "num_hidden_layers", int),
            num_attention_heads=_need(c, "num_attention_heads", int),
            num_key_value_heads=_need(c, "num_key_value_heads", int), head_dim=_need(c, "head_dim", int),
            intermediate_size=_need(c, "intermediate_size", int), rms_norm_eps=_need(c, "rms_norm_eps", float),
            rope_theta=float(_need(rope, "rope_theta", float)),
            tie_word_embeddings=bool(c.get("tie_word_embeddings", False)),
            max_position_embeddings=c.get("max_position_embeddings"), eos_token_ids=eos)
        for name in ("hidden_size", "vocab_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                     "head_dim", "intermediate_size"):
            if getattr(cfg, name) < 1:
                raise ConfigError(f"config.json: {name!r} must be positive")
        if cfg.num_attention_heads % cfg.num_key_value_heads:
            raise ConfigError("config.json: num_attention_heads must be a multiple of num_key_value_heads")
        if cfg.head_dim % 2:
            raise ConfigError("config.json: head_dim must be even (the rotation pairs its halves)")
        return cfg


WEIGHT_RULES = (
    WeightRule("model.embed_tokens.weight", "embed.weight"),
    WeightRule("model.norm.weight", "norm.weight"),
    WeightRule("lm_head.weight", "head.weight"),
    WeightRule("model.layers.{i}.input_layernorm.{rest}", "layers.{i}.input_norm.{rest}"),
    WeightRule("model.layers.{i}.post_attention_layernorm.{rest}", "layers.{i}.post_norm.{rest}"),
    WeightRule("model.layers.{i}.self_attn.{rest}", "layers.{i}.mixer.{rest}"),
    WeightRule("model.layers.{i}.mlp.{rest}", "layers.{i}.ffn.{rest}"),
)


def recipe(cfg: Qwen3Config) -> ModelSpec:
    norm = PartRef.of("norm", "rmsnorm", eps=cfg.rms_norm_eps)
    mixer = PartRef.of("mixer", "gqa", heads=cfg.num_attention_heads, kv_heads=cfg.num_key_value_heads,
                       head_dim=cfg.head_dim, qk_norm=norm, window=0,
                       position=PartRef.of("position", "rope", theta=cfg.rope_theta, rotary_dim=cfg.head_dim))
    ffn = PartRef.of("ffn", "swiglu", inter=cfg.intermediate_size)
    layer = LayerSpec(PartRef.of("block", "prenorm"), mixer, ffn, norm)
    n = cfg.num_hidden_layers
    return ModelSpec(
        hidden=cfg.hidden_size, vocab=cfg.vocab_size, layers=(layer,) * n,
        order=tuple(Run(i, i) for i in range(n)),
        embed=PartRef.of("embed", "table"), norm=norm, head=PartRef.of("head", "linear", tied=cfg.tie_word_embeddings),
        weight_rules=WEIGHT_RULES, ignore_stored=("lm_head.",) if cfg.tie_word_embeddings else ())


register_architecture("Qwen3ForCausalLM", Qwen3Config.from_dict, recipe)
