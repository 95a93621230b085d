"""What every part is made of: parameters with stored names, children, a registry per kind, the build context.

A part knows its own sizes and constants (they are constructor arguments) and the kernels it calls; it does not
know which model it sits in. The reference builds its units the same way, by reference and with injected
parameters (core/holon/core/build.py:36-167).
"""
from __future__ import annotations

import dataclasses
from collections.abc import Callable, Iterator
from typing import Any

import torch

from ..config.spec import PartRef


class Param:
    """One tensor of a part. `pieces` maps a loadable name (relative to the part) to the rows of this tensor that it
    fills: a merged projection lists its stored halves there, a plain tensor lists itself.

    `kind`: "matrix" (a product's weight, stored [out, in], kept in the engine's dtype), "gain" (a norm's weight:
    kept in the engine's dtype unless the file stores 32 bits, which stay 32 bits) or "table" (embedding rows)."""

    def __init__(self, name: str, shape: tuple[int, ...], kind: str, pieces: dict[str, tuple[int, int]] | None = None):
        self.name, self.shape, self.kind = name, tuple(shape), kind
        self.pieces = pieces or {name: (0, self.shape[0])}
        self.tensor: torch.Tensor | None = None

    def __repr__(self) -> str:
        return f"Param({self.name}, {self.shape}, {self.kind})"


class Part:
    def __init__(self) -> None:
        self._params: dict[str, Param] = {}
        self._children: dict[str, "Part"] = {}

    def add_param(self, name: str, shape, kind: str, pieces=None) -> Param:
        if name in self._params:
            raise ValueError(f"parameter {name!r} declared twice")
        self._params[name] = p = Param(name, tuple(shape), kind, pieces)
        return p

    def add_child(self, name: str, part: "Part") -> "Part":
        self._children[name] = part
        return part

    def params(self, prefix: str = "") -> Iterator[tuple[str, Param]]:
        for name, p in self._params.items():
            yield prefix + name, p
        for name, child in self._children.items():
            yield from child.params(f"{prefix}{name}.")

    def loadables(self, prefix: str = "") -> Iterator[tuple[str, Param, tuple[int, int]]]:
        """(qualified loadable name, parameter, rows it fills) of this part and its children."""
        for p in self._params.values():
            for piece, rows in p.pieces.items():
                yield prefix + piece, p, rows
        for name, child in self._children.items():
            yield from child.loadables(f"{prefix}{name}.")

    def finalize(self) -> None:
        """Called once after every parameter holds its tensor. What needs the tensors, the device or the kernel table
        (derived tensors, a library of the part's own: `ctx.kernels.extension`) is done here, not in the constructor:
        a model is also built on no device and without kernels, only to list its parameters."""
        for child in self._children.values():
            child.finalize()


# ---------------------------------------------------------------- what a mixer may ask of the cache manager

@dataclasses.dataclass(frozen=True)
class PagedKV:
    """Keys and values of every token, in pages; `window` W > 0: only the last W positions are ever read again, so
    pages that lie wholly before them are given back."""

    kv_heads: int
    head_dim: int
    window: int = 0


@dataclasses.dataclass(frozen=True)
class SlotState:
    """State of fixed size per request: one tensor [requests + 1, *shape] per layer that declares it, zeroed when a
    request takes the slot. `chunk` > 1: the mixer updates this state in chunks of that many tokens, so a prompt may
    be cut only at positions that are multiples of it (the scheduler shortens a portion to the last such position;
    the portion that ends the prompt ends where the prompt ends), as the reference cuts where a recurrent state wants
    its checkpoints (core/holon/core/sched.py:150; core/holon/core/state.py:311-318)."""

    name: str
    shape: tuple[int, ...]
    dtype: str = "float32"
    chunk: int = 1


# ---------------------------------------------------------------- registries

_REGISTRIES: dict[str, dict[str, Callable[..., Part]]] = {
    k: {} for k in ("mixer", "ffn", "norm", "position", "block", "embed", "head")}


def register_part(kind: str, name: str, factory: Callable[..., Part], replace: bool = False) -> None:
    """`factory(ctx, **ref parameters, **site arguments) -> Part`."""
    if kind not in _REGISTRIES:
        raise ValueError(f"no registry of kind {kind!r}; kinds: {sorted(_REGISTRIES)}")
    if name in _REGISTRIES[kind] and not replace:
        raise ValueError(f"{kind} {name!r} is registered already")
    _REGISTRIES[kind][name] = factory


def unregister_part(kind: str, name: str) -> None:
    _REGISTRIES[kind].pop(name, None)


class BuildContext:
    """What parts see while they are built: device, dtype, the kernel table and the engine's limits."""

    def __init__(self, device, dtype: torch.dtype, kernels, max_positions: int, max_step_tokens: int = 0) -> None:
        self.device, self.dtype, self.kernels = torch.device(device), dtype, kernels
        self.max_positions, self.max_step_tokens = max_positions, max_step_tokens

    def part(self, ref: PartRef, **site: Any) -> Part:
        from . import _builtin  # noqa: F401  (registers the built-in parts)
        try:
            factory = _REGISTRIES[ref.kind][ref.name]
        except KeyError:
            known = sorted(_REGISTRIES.get(ref.kind, {}))
            raise KeyError(f"no {ref.kind} named {ref.name!r}; registered: {known}") from None
        return factory(self, **ref.kwargs(), **site)

    def empty(self, *shape: int, dtype: torch.dtype | None = None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)


class Residual:
    """The residual stream between blocks: `h` [T, H] in 32-bit, and `delta`, a part's output that has not been
    added yet. The next norm adds it while it normalises, in one kernel. Or the product that ended the part has
    added its output itself and left the next norm's rows behind (`normed`, made with the weight of `normed_by`):
    then that norm has nothing left to launch."""

    __slots__ = ("h", "delta", "normed", "normed_by")

    def __init__(self, h: torch.Tensor, delta: torch.Tensor | None = None) -> None:
        self.h, self.delta = h, delta
        self.normed, self.normed_by = None, None


class Scaled:
    """Rows of a norm that still lack their row scale: `y` [T, dim] = stream · (weight + offset) in the engine's
    dtype, and `ss` [parts, 16] float32, partial sums of squares of the stream per token (16 to a part, unused ones 0).
    x = y · rsqrt(sum(ss) / dim + eps) row by row; a product that takes these rows applies the scale to its sums
    instead, since (y · s) · Wᵀ = (y · Wᵀ) · s. Only parts that say `takes_scaled` are handed one."""

    __slots__ = ("y", "ss", "eps", "dim")

    def __init__(self, y: torch.Tensor, ss: torch.Tensor, eps: float, dim: int) -> None:
        self.y, self.ss, self.eps, self.dim = y, ss, eps, dim

    @property
    def shape(self):
        return self.y.shape

    @property
    def dtype(self):
        return self.y.dtype


class Link:
    """An offer to the product that ends a mixer or a feed-forward: add your output into `stream` yourself and leave
    the rows of `norm` behind (`Linear.forward(x, link=...)`). A part that takes it from `step.link` returns None in
    place of its output; a part that knows nothing of it returns its output as ever."""

    __slots__ = ("stream", "norm")

    def __init__(self, stream: Residual, norm) -> None:
        self.stream, self.norm = stream, norm


def take_link(step):
    """The block's offer for the product that ends the part that calls this (None: there is none); taken, it is gone
    from the step, which is how the block sees that the part has used it."""
    link = getattr(step, "link", None)
    if link is not None:
        step.link = None
    return link
