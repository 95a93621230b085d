"""RMSNorm: x · rsqrt(mean(x²) + eps) · (weight + offset), all in 32-bit, one rounding at the end
(std/holon_std/ops/units.py:16-35; formula std/holon_std/ops/reference.py:7-18)."""
from __future__ import annotations

import torch

from .base import BuildContext, Part, Residual


class RMSNorm(Part):
    def __init__(self, ctx: BuildContext, *, eps: float, dim: int, offset: float = 0.0) -> None:
        super().__init__()
        self.ctx, self.eps, self.dim, self.offset = ctx, float(eps), dim, float(offset)
        self.weight = self.add_param("weight", (dim,), "gain")

    def apply(self, x: torch.Tensor) -> torch.Tensor:
        """The norm of the rows of `x` [rows, dim] (engine dtype or 32-bit), as a new tensor of the engine's dtype."""
        out = self.ctx.empty(*x.shape)
        self.ctx.kernels.rmsnorm(out, x, self.weight.tensor, self.eps, self.offset)
        return out

    def add(self, stream: Residual) -> torch.Tensor:
        """Adds the stream's pending output into it and returns the norm of the sum; or, where the product before
        has done both, the rows it left (base.Scaled)."""
        if stream.normed is not None:
            rows, by, stream.normed, stream.normed_by = stream.normed, stream.normed_by, None, None
            if by is self:
                return rows                                # (made for another norm: dropped, the stream itself is whole)
        out = self.ctx.empty(*stream.h.shape)
        self.ctx.kernels.add_rmsnorm(out, stream.h, stream.delta, self.weight.tensor, self.eps, self.offset, None)
        stream.delta = None
        return out

    def gather(self, stream: Residual, index: torch.Tensor) -> torch.Tensor:
        """The norm of rows `index` of the stream (pending output included); the stream is left as it is."""
        out = self.ctx.empty(index.shape[0], self.dim)
        self.ctx.kernels.add_rmsnorm(out, stream.h, stream.delta, self.weight.tensor, self.eps, self.offset, index)
        return out
