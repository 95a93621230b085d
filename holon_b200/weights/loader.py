"""Binding stored tensors to the model's parameters by name.

Names are mapped by the recipe's rules (`{i}` a layer number, `{rest}` any tail, whole-name matches:
core/holon/core/build.py:317-337). Every loadable name must be filled exactly once; several stored tensors may fill
the rows of one parameter (merged projections, build.py:372-424 with std/holon_std/ops/units.py:253-277). Faults do
not stop at the first one: one `WeightError` lists the missing names, the unexpected ones and the wrong shapes.

Precision: products' weights and tables take the engine's dtype; a norm weight that the file stores in 32 bits stays
32-bit even under a bfloat16 engine; integer tensors become int32.
"""
from __future__ import annotations

import re
from collections.abc import Iterable

import torch

from ..config.spec import ModelSpec, WeightRule


class WeightError(ValueError):
    def __init__(self, missing, unexpected, shapes, twice=()) -> None:
        self.missing, self.unexpected, self.shapes, self.twice = list(missing), list(unexpected), list(shapes), list(twice)
        lines = ["the stored tensors do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.twice:
            lines.append(f"  stored twice ({len(self.twice)}): " + ", ".join(self.twice))
        for name, got, want in self.shapes:
            lines.append(f"  wrong shape: {name} is {tuple(got)}, the model needs {tuple(want)}")
        super().__init__("\n".join(lines))


def _regex(template: str) -> re.Pattern:
    parts = re.split(r"(\{i\}|\{rest\})", template)
    out = "".join({"{i}": r"(?P<i>\d+)", "{rest}": r"(?P<rest>.+)"}.get(p, re.escape(p)) for p in parts)
    return re.compile(out + r"\Z")


class NameMap:
    """Both directions of the rules: `ours(stored)` and `stored(ours)`; None where no rule matches."""

    def __init__(self, rules: Iterable[WeightRule]) -> None:
        self.rules = [(_regex(r.stored), r.ours, _regex(r.ours), r.stored) for r in rules]

    @staticmethod
    def _apply(pattern: re.Pattern, template: str, name: str) -> str | None:
        m = pattern.match(name)
        return template.format(**m.groupdict()) if m else None

    def ours(self, stored: str) -> str | None:
        for pattern, template, _, _ in self.rules:
            if (out := self._apply(pattern, template, stored)) is not None:
                return out
        return None

    def stored(self, ours: str) -> str | None:
        for _, _, pattern, template in self.rules:
            if (out := self._apply(pattern, template, ours)) is not None:
                return out
        return None


def _dtype_for(kind: str, stored: torch.dtype, engine: torch.dtype) -> torch.dtype:
    if not stored.is_floating_point:
        return torch.int32
    if kind == "gain" and stored == torch.float32:
        return torch.float32
    return engine


def load_weights(model, spec: ModelSpec, tensors: Iterable[tuple[str, torch.Tensor]], dtype: torch.dtype,
                 device) -> int:
    """Fills every parameter of `model` from (stored name, tensor) pairs; returns the bytes now held on `device`."""
    names = NameMap(spec.weight_rules)
    targets = {name: (p, rows) for name, p, rows in model.loadables()}
    filled: set[str] = set()
    unexpected, shapes, twice = [], [], []
    for stored, tensor in tensors:
        if any(stored.startswith(prefix) for prefix in spec.ignore_stored):
            continue
        ours = names.ours(stored)
        if ours is None or ours not in targets:
            unexpected.append(stored)
            continue
        if ours in filled:
            twice.append(stored)
            continue
        p, (r0, r1) = targets[ours]
        want = (r1 - r0, *p.shape[1:])
        if tuple(tensor.shape) != want:
            shapes.append((stored, tensor.shape, want))
            filled.add(ours)                     # it is there, only wrong: not also "missing"
            continue
        if p.tensor is None:
            p.tensor = torch.empty(p.shape, dtype=_dtype_for(p.kind, tensor.dtype, dtype), device=device)
        p.tensor[r0:r1].copy_(tensor)
        filled.add(ours)
    missing = [names.stored(n) or n for n in targets if n not in filled]
    if missing or unexpected or shapes or twice:
        raise WeightError(missing, unexpected, shapes, twice)
    model.finalize()
    return sum(p.tensor.numel() * p.tensor.element_size() for _, p in model.params())
