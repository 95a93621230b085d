"""Token embedding (a row gather, no scaling) and the output head (logits in 32-bit; a tied head reads the
embedding's table) (std/holon_std/ops/units.py:280-348)."""
from __future__ import annotations

import torch

from .base import BuildContext, Part, Residual


class Embedding(Part):
    def __init__(self, ctx: BuildContext, *, vocab: int, hidden: int) -> None:
        super().__init__()
        self.ctx, self.vocab, self.hidden = ctx, vocab, hidden
        self.weight = self.add_param("weight", (vocab, hidden), "table")

    def forward(self, ids: torch.Tensor) -> Residual:
        h = self.ctx.empty(ids.shape[0], self.hidden, dtype=torch.float32)
        self.ctx.kernels.embed(h, self.weight.tensor, ids)
        return Residual(h)


class Head(Part):
    def __init__(self, ctx: BuildContext, *, vocab: int, hidden: int, tied: bool, embed: Embedding | None) -> None:
        super().__init__()
        self.ctx, self.vocab = ctx, vocab
        if tied and embed is None:
            raise ValueError("a tied head needs the embedding")
        self._embed = embed if tied else None
        self.weight = None if tied else self.add_param("weight", (vocab, hidden), "matrix")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w = self._embed.weight.tensor if self._embed is not None else self.weight.tensor
        logits = self.ctx.empty(x.shape[0], self.vocab, dtype=torch.float32)
        self.ctx.kernels.linear(logits, x, w)
        return logits
