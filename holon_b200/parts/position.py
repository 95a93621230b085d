"""Position encodings. A position encoding hands its mixer a table of angles' cosines and sines per position;
the mixer's fused kernel rotates q and k with it.

Rope: inv_freq_i = θ^(−2i/rotary_dim), angle = position · inv_freq in 32-bit, half-split pairs (i, i + rotary_dim/2);
dimensions past `rotary_dim` pass through (std/holon_std/ops/units.py:38-63; std/holon_std/ops/reference.py:21-30).
"""
from __future__ import annotations

import torch

from .base import BuildContext, Part


class Rope(Part):
    def __init__(self, ctx: BuildContext, *, theta: float, rotary_dim: int, head_dim: int) -> None:
        super().__init__()
        if rotary_dim % 2 or not 0 <= rotary_dim <= head_dim:
            raise ValueError(f"rope: rotary_dim {rotary_dim} must be even and at most head_dim {head_dim}")
        self.theta, self.rotary_dim = float(theta), rotary_dim
        self.table = self.angles(ctx.max_positions).to(ctx.device)

    def angles(self, positions: int) -> torch.Tensor:
        """[positions, rotary_dim] 32-bit: cosines of the rotary_dim/2 angles, then their sines."""
        rd = self.rotary_dim
        inv_freq = 1.0 / (self.theta ** (torch.arange(0, rd, 2, dtype=torch.float32) / rd))
        angle = torch.arange(positions, dtype=torch.float32)[:, None] * inv_freq[None, :]
        return torch.cat((angle.cos(), angle.sin()), dim=-1).contiguous()
