"""Pre-norm residual block: h += mixer(input_norm(h)); h += ffn(post_norm(h))
(std/holon_std/blocks/units.py:8-25). The sums are folded into the next norm's kernel: the block leaves the
feed-forward's output pending on the stream."""
from __future__ import annotations

from ..config.spec import PartRef
from .base import BuildContext, Part, Residual


class PreNorm(Part):
    def __init__(self, ctx: BuildContext, *, layer: int, hidden: int, mixer: PartRef, ffn: PartRef,
                 norm: PartRef) -> None:
        super().__init__()
        self.input_norm = self.add_child("input_norm", ctx.part(norm, dim=hidden))
        self.mixer = self.add_child("mixer", ctx.part(mixer, layer=layer, hidden=hidden))
        self.post_norm = self.add_child("post_norm", ctx.part(norm, dim=hidden))
        self.ffn = self.add_child("ffn", ctx.part(ffn, layer=layer, hidden=hidden))

    def forward(self, stream: Residual, step, cache) -> Residual:
        x = self.input_norm.add(stream)
        stream.delta = self.mixer.forward(x, step, cache)
        x = self.post_norm.add(stream)
        stream.delta = self.ffn.forward(x, step)
        return stream
