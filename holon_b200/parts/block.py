"""Pre-norm residual block: h += mixer(input_norm(h)); h += ffn(post_norm(h))
(std/holon_std/blocks/units.py:8-25). The sums are folded into the next norm's kernel: the block leaves the
feed-forward's output pending on the stream. For the few rows of a decode step sum and norm move one kernel further
up, into the product that ends the mixer or the feed-forward (base.Link, base.Scaled)."""
from __future__ import annotations

from ..config.spec import PartRef
from .base import BuildContext, Link, Part, Residual


class PreNorm(Part):
    def __init__(self, ctx: BuildContext, *, layer: int, hidden: int, mixer: PartRef, ffn: PartRef,
                 norm: PartRef) -> None:
        super().__init__()
        self.ctx = ctx
        self.input_norm = self.add_child("input_norm", ctx.part(norm, dim=hidden))
        self.mixer = self.add_child("mixer", ctx.part(mixer, layer=layer, hidden=hidden))
        self.post_norm = self.add_child("post_norm", ctx.part(norm, dim=hidden))
        self.ffn = self.add_child("ffn", ctx.part(ffn, layer=layer, hidden=hidden))

    def forward(self, stream: Residual, step, cache, after=None) -> Residual:
        """`after`: the block that runs next (None: none, or unknown). For the few rows of a decode step the
        product that ends the mixer does the residual sum and the post norm in its epilogue, and the one that ends
        the feed-forward the sum and `after`'s input norm (see base.Link), where the part that reads those rows can
        take them unscaled."""
        x = self.input_norm.add(stream)
        step.link = self._offer(stream, step, self.post_norm, self.ffn)
        stream.delta = self.mixer.forward(x, step, cache)
        step.link = None                                             # (an offer nobody took lapses)
        x = self.post_norm.add(stream)
        step.link = self._offer(stream, step, getattr(after, "input_norm", None), getattr(after, "mixer", None))
        stream.delta = self.ffn.forward(x, step)
        step.link = None
        return stream

    def _offer(self, stream, step, norm, reader):
        can = getattr(self.ctx.kernels, "can_link", None)
        if can is None or not getattr(reader, "takes_scaled", False) or not hasattr(norm, "weight"):
            return None
        return Link(stream, norm) if can(step.rows.n_tokens, stream.h.shape[1], norm) else None
