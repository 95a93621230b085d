"""What a recipe hands to the builder: a model described as data.

A `PartRef` names a registered part and its parameters; a `LayerSpec` names the block, mixer, feed-forward and
norm of one layer; `ModelSpec.order` lists the runs of a step: which layer runs, which cache entry it uses and
whether it fills that entry or only reads what another run filled. The builder (`holon_b200.parts.model`)
turns this into parts; nothing here imports torch.

The reference keeps the same split between a pure recipe and built units (core/holon/api/model.py:27-81,
core/holon/api/terms.py:23-62).
"""
from __future__ import annotations

import dataclasses
from typing import Any


@dataclasses.dataclass(frozen=True)
class PartRef:
    """`kind` is the registry ("mixer", "ffn", "norm", "position", "block", "embed", "head"), `name` the part."""

    kind: str
    name: str
    params: tuple[tuple[str, Any], ...] = ()

    @staticmethod
    def of(kind: str, name: str, **params: Any) -> "PartRef":
        return PartRef(kind, name, tuple(sorted(params.items())))

    def kwargs(self) -> dict[str, Any]:
        return dict(self.params)


@dataclasses.dataclass(frozen=True)
class LayerSpec:
    block: PartRef
    mixer: PartRef
    ffn: PartRef
    norm: PartRef


@dataclasses.dataclass(frozen=True)
class Run:
    """One entry of the run order: layer `layer` runs with cache entry `cache`; `fills` says whether this run
    writes the step's tokens into the entry (the entry's owner) or only reads what an earlier run wrote."""

    layer: int
    cache: int
    fills: bool = True


@dataclasses.dataclass(frozen=True)
class WeightRule:
    """`stored` and `ours` are name templates with `{i}` (a layer number) and `{rest}` (any tail)."""

    stored: str
    ours: str


@dataclasses.dataclass(frozen=True)
class ModelSpec:
    hidden: int
    vocab: int
    layers: tuple[LayerSpec, ...]
    order: tuple[Run, ...]
    embed: PartRef
    norm: PartRef
    head: PartRef
    weight_rules: tuple[WeightRule, ...]
    ignore_stored: tuple[str, ...] = ()          # stored-name prefixes that are skipped (a tied head's copy)

    def __post_init__(self) -> None:
        filled: set[int] = set()
        for run in self.order:
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"run order names layer {run.layer}, the model has {len(self.layers)}")
            if run.fills:
                if run.cache in filled:
                    raise ValueError(f"cache entry {run.cache} is filled by two runs")
                filled.add(run.cache)
            elif run.cache not in filled:
                raise ValueError(f"layer {run.layer} reads cache entry {run.cache} before any run fills it")
