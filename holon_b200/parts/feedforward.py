"""SwiGLU: down(silu(gate(x)) · up(x)), gate and up in one product with gate's rows first, silu in 32-bit
(std/holon_std/ffn/units.py:12-50; std/holon_std/ffn/reference.py:7-12)."""
from __future__ import annotations

import torch

from .base import BuildContext, Part, take_link
from .linear import Linear


class SwiGLU(Part):
    def __init__(self, ctx: BuildContext, *, inter: int, hidden: int, layer: int = 0) -> None:
        super().__init__()
        self.ctx, self.inter = ctx, inter
        self.gate_up = self.add_child("gate_up", Linear(ctx, "weight", hidden, {
            "gate_proj.weight": inter, "up_proj.weight": inter}))
        self.down = self.add_child("down_proj", Linear(ctx, "weight", inter, {"weight": hidden}))

    def loadables(self, prefix: str = ""):
        for name, p, rows in super().loadables(prefix):
            yield name.replace(prefix + "gate_up.", prefix, 1), p, rows

    takes_scaled = True                      # x may be base.Scaled: the first product applies the row scale

    def forward(self, x: torch.Tensor, step) -> torch.Tensor | None:
        act = self.ctx.empty(x.shape[0], self.inter)
        self.ctx.kernels.swiglu_gate_up(act, x, self.gate_up.weight.tensor)
        return self.down.forward(act, link=take_link(step))
