"""Grouped-query attention over a paged cache.

qkv = x·Wqkvᵀ in one product; per head RMSNorm of q and k (optional), rotation, keys and values written to the
step's pages, attention of the new rows over everything the request holds, output projection
(std/holon_std/mixers/gqa/units.py:108-294; formulas std/holon_std/mixers/gqa/reference.py:26-60, 91-101).
Query head h reads KV head h // (heads / kv_heads); a query at position p sees keys j ≤ p, and with a window W > 0
only those with p − j < W.
"""
from __future__ import annotations

import torch

from ..config.spec import PartRef
from .base import BuildContext, PagedKV, Part, take_link
from .linear import Linear


class GQA(Part):
    def __init__(self, ctx: BuildContext, *, heads: int, kv_heads: int, head_dim: int, hidden: int,
                 position: PartRef | None, qk_norm: PartRef | None = None, window: int = 0, layer: int = 0) -> None:
        super().__init__()
        if heads % kv_heads:
            raise ValueError(f"gqa: {heads} heads are no multiple of {kv_heads} kv heads")
        self.ctx, self.heads, self.kv_heads, self.head_dim, self.window = ctx, heads, kv_heads, head_dim, int(window)
        self.scale = 1.0 / head_dim ** 0.5
        self.qkv = self.add_child("qkv", Linear(ctx, "weight", hidden, {
            "q_proj.weight": heads * head_dim, "k_proj.weight": kv_heads * head_dim,
            "v_proj.weight": kv_heads * head_dim}))
        self.o_proj = self.add_child("o_proj", Linear(ctx, "weight", heads * head_dim, {"weight": hidden}))
        self.q_norm = self.k_norm = None
        if qk_norm is not None:
            self.q_norm = self.add_child("q_norm", ctx.part(qk_norm, dim=head_dim))
            self.k_norm = self.add_child("k_norm", ctx.part(qk_norm, dim=head_dim))
        self.position = self.add_child("position", ctx.part(position, head_dim=head_dim)) if position else None

    # the loadable names of the merged product are the stored ones, without the child's own prefix
    def loadables(self, prefix: str = ""):
        for name, p, rows in super().loadables(prefix):
            yield name.replace(prefix + "qkv.", prefix, 1), p, rows

    takes_scaled = True                      # x may be base.Scaled: both first products apply the row scale

    def cache(self) -> PagedKV:
        return PagedKV(self.kv_heads, self.head_dim, self.window)

    def slot_states(self):
        return ()

    @property
    def plan_group(self):
        """Mixers with equal answers here plan a captured step alike: one of them is asked."""
        return "gqa", self.heads, self.kv_heads, self.head_dim, self.window

    def capture_plan(self, step, max_model_len: int):
        """What the attention kernels pin for a step that is captured as a CUDA graph (see base.Part)."""
        plan = getattr(self.ctx.kernels, "attention_capture_plan", None)
        return plan(step.rows, max_model_len) if plan is not None else None

    def forward(self, x: torch.Tensor, step, cache) -> torch.Tensor:
        t, k = x.shape[0], self.ctx.kernels
        q = self.ctx.empty(t, self.heads, self.head_dim)
        norm, pos = self.q_norm, self.position
        after = (step.positions, pos.table if pos else None, pos.rotary_dim if pos else 0,
                 norm.weight.tensor if norm else None, self.k_norm.weight.tensor if norm else None,
                 norm.eps if norm else 0.0, norm.offset if norm else 0.0,
                 cache.kv if cache.fills else None, cache.group.write_index if cache.fills else None,
                 self.heads, self.kv_heads, self.head_dim)
        fused = getattr(k, "qkv_rope", None)                         # a kernel table may do the product and what follows in one
        if fused is None or not fused(q, x, self.qkv.weight.tensor, *after):
            k.qk_norm_rope_kv_write(q, self.qkv.forward(x), *after)
        o = self.ctx.empty(t, self.heads, self.head_dim)
        k.paged_attention(o, q, cache.kv, cache.group.block_table, step.rows, self.scale, self.window)
        return self.o_proj.forward(o.view(t, self.heads * self.head_dim), link=take_link(step))
