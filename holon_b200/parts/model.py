"""A model put together from a `ModelSpec`: embedding → the runs of the order list → final norm → head
(core/holon/core/build.py:273-314). It also works out which cache entries the runs need and which of them may share
pages: entries whose mixers ask for the same thing form one group."""
from __future__ import annotations

import dataclasses

import torch

from ..config.spec import ModelSpec
from .base import BuildContext, PagedKV, Part, SlotState


@dataclasses.dataclass(frozen=True)
class CacheEntry:
    """One cache entry of the run order: which layer fills it and what that layer's mixer asked for."""

    entry: int
    layer: int
    decl: PagedKV | None
    slot_states: tuple[SlotState, ...]


class LayerCache:
    """What a mixer gets for one run: its entry's pages (`kv`), the step's data of the entry's group (`group`: block
    table, write index), whether this run fills the entry, and its slot-state tensors by name."""

    __slots__ = ("kv", "group", "fills", "slots")

    def __init__(self, kv, group, fills: bool, slots: dict[str, torch.Tensor]) -> None:
        self.kv, self.group, self.fills, self.slots = kv, group, fills, slots


class Model(Part):
    def __init__(self, spec: ModelSpec, ctx: BuildContext) -> None:
        super().__init__()
        self.spec, self.ctx = spec, ctx
        self.embed = self.add_child("embed", ctx.part(spec.embed, vocab=spec.vocab, hidden=spec.hidden))
        self.layers = []
        built: dict = {}
        for i, layer in enumerate(spec.layers):
            block = ctx.part(layer.block, layer=i, hidden=spec.hidden, mixer=layer.mixer, ffn=layer.ffn,
                             norm=layer.norm)
            self.layers.append(self.add_child(f"layers.{i}", block))
        self.norm = self.add_child("norm", ctx.part(spec.norm, dim=spec.hidden))
        self.head = self.add_child("head", ctx.part(spec.head, vocab=spec.vocab, hidden=spec.hidden, embed=self.embed))
        self.entries = self._entries()
        planners: dict = {}                                   # one mixer of each kind that plans captured steps
        for layer in self.layers:
            mixer = getattr(layer, "mixer", None)
            if hasattr(mixer, "capture_plan"):
                planners.setdefault(getattr(mixer, "plan_group", id(mixer)), mixer)
        self._planners = tuple(planners.values())

    def _entries(self) -> tuple[CacheEntry, ...]:
        entries: dict[int, CacheEntry] = {}
        for run in self.spec.order:
            mixer = self.layers[run.layer].mixer
            decl, slots = mixer.cache(), tuple(mixer.slot_states())
            if run.fills:
                entries[run.cache] = CacheEntry(run.cache, run.layer, decl, slots)
            elif entries[run.cache].decl != decl:
                raise ValueError(f"layer {run.layer} reads cache entry {run.cache}, filled by layer "
                                 f"{entries[run.cache].layer} with other sizes: {entries[run.cache].decl} vs {decl}")
        return tuple(entries[k] for k in sorted(entries))

    def capture_plan(self, step, max_model_len: int) -> tuple:
        """A step that is to run as a CUDA graph is replayed for every later step of the same shape: whatever a
        mixer's kernels decide from the rows' lengths on the host (how keys are shared out over CTAs, how many tiles a
        launch has) is frozen at the capture. Each mixer that makes such decisions answers `capture_plan(step,
        max_model_len)`: it pins them on the step in a form that serves every step with the same answer, and returns
        that answer, hashable. The answers of all mixers are part of the graph's key, so a step whose rows call for
        another plan gets another graph (core/holon/api/mixer.py:20-28 splits a mixer's planning the same way, into
        bounds known on the host and metadata made on the device)."""
        return tuple(mixer.capture_plan(step, max_model_len) for mixer in self._planners)

    def trunk(self, step):
        """The residual stream after the last run, for every token of the step."""
        stream = self.embed.forward(step.token_ids)
        order = self.spec.order
        for i, run in enumerate(order):
            after = self.layers[order[i + 1].layer] if i + 1 < len(order) else None
            stream = self.layers[run.layer].forward(stream, step, step.layer_cache(run), after)
        flush = getattr(self.ctx.kernels, "flush", None)
        if flush is not None:                          # a kernel table may queue launches: the stream is whole from here on
            flush()
        return stream

    def forward(self, step) -> torch.Tensor | None:
        """Logits [R, V] in 32-bit at the step's wanted places; None if the step wants none (the head is skipped)."""
        return self.logits_at(self.trunk(step), step.logits_index)

    def logits_at(self, stream, index: torch.Tensor) -> torch.Tensor | None:
        """Logits [R, V] in 32-bit of the step's tokens `index` (int32 [R]) from the trunk's residual stream."""
        if index.shape[0] == 0:
            return None
        return self.head.forward(self.norm.gather(stream, index))
