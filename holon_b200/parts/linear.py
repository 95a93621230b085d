"""y = x · Wᵀ with W stored [out, in] and no bias (std/holon_std/ops/units.py:189-277). Several stored tensors
may fill the rows of one weight, so that one product serves them all (the reference's `merge`)."""
from __future__ import annotations

import torch

from .base import BuildContext, Part


class Linear(Part):
    def __init__(self, ctx: BuildContext, name: str, width_in: int, pieces: dict[str, int]) -> None:
        """`pieces`: loadable name -> rows, in the order they are stacked."""
        super().__init__()
        self.ctx, self.width_in = ctx, width_in
        rows, at = {}, 0
        for piece, n in pieces.items():
            rows[piece], at = (at, at + n), at + n
        self.width_out = at
        self.weight = self.add_param(name, (at, width_in), "matrix", rows)

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype | None = None, link=None) -> torch.Tensor | None:
        """x · Wᵀ. With `link` (base.Link): the product is added into the link's stream, the rows of the link's norm
        are left on the stream, and None is returned; where the kernel table has no such product for these sizes, the
        plain product is returned as ever."""
        if link is not None:
            stream, norm = link.stream, link.norm
            rows = self.ctx.kernels.linear_link(stream.h, x, self.weight.tensor, norm.weight.tensor, norm.eps, norm.offset)
            if rows is not None:                           # (None: that kernel does not take these sizes or this dtype)
                stream.normed, stream.normed_by = rows, norm
                return None
        out = self.ctx.empty(x.shape[0], self.width_out, dtype=out_dtype)
        self.ctx.kernels.linear(out, x, self.weight.tensor)
        return out
