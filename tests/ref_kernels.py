"""Every kernel of the engine as plain torch code on the CPU, one function per kernel, same arguments.

Two uses. The `-m gpu` tests compare each CUDA kernel with its function here, at sizes of their own. And the
`-m "not gpu"` tests hand this table to the engine in place of the CUDA one, so that the host side (batch layout,
cache, scheduler) runs on a machine without a GPU. The product never loads this file; mxinO/holon keeps its CPU
oracle kernels test-only in the same way (testing/holon_testing/ref_kernels/plugin.py:24-35).
Formulas: std/holon_std/ops/reference.py:7-30, std/holon_std/mixers/gqa/reference.py:26-60 and 91-101,
std/holon_std/ffn/reference.py:7-12, std/holon_std/sampling/sampler.py:24-61.
"""
from __future__ import annotations

import torch

_M32 = 0xFFFFFFFF


def _mix32(x):
    x = x ^ (x >> 16)
    x = (x * 0x7FEB352D) & _M32
    x = x ^ (x >> 15)
    x = (x * 0x846CA68B) & _M32
    return x ^ (x >> 16)


class RefKernels:
    name = "reference (torch, CPU)"

    def embed(self, out, table, ids):
        out.copy_(table[ids.long()].float())

    def rmsnorm(self, out, x, weight, eps, offset):
        x = x.float()
        out.copy_((x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * (weight.float() + offset)).to(out.dtype))

    def add_rmsnorm(self, out, h, delta, weight, eps, offset, index):
        rows = slice(None) if index is None else index.long()
        v = h[rows] if delta is None else h[rows] + delta[rows].float()
        if index is None and delta is not None:
            h.copy_(v)
        self.rmsnorm(out, v, weight, eps, offset)

    def qk_norm_rope_kv_write(self, q_out, qkv, positions, table, rotary_dim, q_weight, k_weight, eps, offset, kv,
                              write_index, heads, kv_heads, head_dim):
        t, dt = qkv.shape[0], qkv.dtype
        q, k, v = qkv.split([heads * head_dim, kv_heads * head_dim, kv_heads * head_dim], dim=-1)
        q, k, v = q.reshape(t, heads, head_dim), k.reshape(t, kv_heads, head_dim), v.reshape(t, kv_heads, head_dim)

        def prepare(x, weight):
            x = x.float()
            if weight is not None:
                x = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * (weight.float() + offset)
                x = x.to(dt).float()
            if rotary_dim:
                half = rotary_dim // 2
                cs = table[positions.long()]
                cos, sin = cs[:, None, :half], cs[:, None, half:]
                a, b, rest = x[..., :half], x[..., half:rotary_dim], x[..., rotary_dim:]
                x = torch.cat((a * cos - b * sin, b * cos + a * sin, rest), dim=-1)
            return x.to(dt)

        q_out.copy_(prepare(q, q_weight))
        if kv is not None:
            k = prepare(k, k_weight)
            page_size = kv.shape[3]
            w = write_index.long()
            ok = w >= 0
            page, off = w[ok] // page_size, w[ok] % page_size
            kv[page, 0, :, off] = k[ok]
            kv[page, 1, :, off] = v[ok]

    def paged_attention(self, out, q, kv, block_table, rows, scale, window):
        page_size, hq, hkv = kv.shape[3], q.shape[1], kv.shape[2]
        out.zero_()
        qs, slots, lens = rows.query_start.tolist(), rows.row_slot.tolist(), rows.kv_len.tolist()
        for b in range(rows.n_rows):
            s, e, n = qs[b], qs[b + 1], lens[b]
            if n == 0 or s == e:
                continue
            pages = block_table[slots[b], : -(-n // page_size)].long()
            k, v = (kv[pages, i].transpose(1, 2).reshape(-1, hkv, kv.shape[4])[:n].float()
                    .repeat_interleave(hq // hkv, dim=1) for i in (0, 1))
            scores = torch.einsum("qhd,khd->hqk", q[s:e].float(), k) * scale
            pos = torch.arange(n - (e - s), n)[:, None]
            key = torch.arange(n)[None, :]
            hidden = key > pos
            if window > 0:
                hidden = hidden | (pos - key >= window)
            probs = scores.masked_fill(hidden, float("-inf")).softmax(-1)
            out[s:e] = torch.einsum("hqk,khd->qhd", probs, v).to(out.dtype)

    def silu_mul(self, out, gate_up):
        gate, up = gate_up.float().chunk(2, dim=-1)
        out.copy_((torch.nn.functional.silu(gate) * up).to(out.dtype))

    def swiglu_gate_up(self, out, x, weight):
        gate_up = torch.empty(x.shape[0], weight.shape[0], dtype=x.dtype)
        self.linear(gate_up, x, weight)
        self.silu_mul(out, gate_up)

    def linear(self, out, x, weight):
        out.copy_((x.float() @ weight.float().T).to(out.dtype))

    def feed_tokens(self, token_ids, last_tokens, rows, from_last):
        for r in range(rows.n_rows):
            if int(from_last[r]):
                token_ids[int(rows.query_start[r])] = last_tokens[int(rows.row_slot[r])]

    def scatter_rows(self, table, slots, rows):
        table[slots.long()] = rows.view(slots.shape[0], table.shape[1])

    def store_tokens(self, last_tokens, slots, tokens, n):
        last_tokens[slots[:n].long()] = tokens[:n]

    def logprobs(self, chosen, top_ids, top, logits, tokens):
        """log softmax of the raw logits: the given token's, and the k most likely ranked (equal ones by ascending id)."""
        k = top.shape[1]
        for r in range(logits.shape[0]):
            lp = logits[r].double().log_softmax(-1)
            chosen[r] = lp[int(tokens[r])]
            order = torch.tensor(sorted(range(lp.numel()), key=lambda i: (-float(lp[i]), i))[:k], dtype=torch.long)
            top_ids[r] = order.to(torch.int32)
            top[r] = lp[order].float()

    def sample(self, tokens, logits, temperature, top_k, top_p, min_p, seed_lo, seed_hi, position, filtered):
        """temperature 0: arg max. Else softmax(logits / T) filtered by top-k, top-p, min-p, drawn by inverse CDF in
        vocabulary order with the uniform of (seed, position)."""
        for r in range(logits.shape[0]):
            t = float(temperature[r])
            if t == 0:
                tokens[r] = int(logits[r].argmax())
                continue
            x = logits[r].double() / t
            keep = torch.ones_like(x, dtype=torch.bool)
            if filtered:
                order = x.argsort(descending=True, stable=True)
                if int(top_k[r]) > 0:
                    keep[order[int(top_k[r]):]] = False
                q = torch.where(keep, x, float("-inf")).softmax(-1)
                if float(top_p[r]) < 1:
                    sq = q[order]
                    keep[order[sq.cumsum(-1) - sq > float(top_p[r])]] = False
                if float(min_p[r]) > 0:
                    keep &= q >= float(min_p[r]) * q.max()
            q = torch.where(keep, x, float("-inf")).softmax(-1)
            lo, hi, pos = int(seed_lo[r]) & _M32, int(seed_hi[r]) & _M32, int(position[r]) & _M32
            h = _mix32(_mix32(lo) ^ hi ^ _mix32(pos))
            u = min(float((torch.tensor(float(h >> 8), dtype=torch.float32) + 0.5) * 2.0 ** -24), 1 - 2.0 ** -24)
            c = q.cumsum(-1)
            i = int(torch.searchsorted(c, torch.tensor([u * float(c[-1])], dtype=c.dtype), right=True)[0])
            tokens[r] = min(i, q.numel() - 1)
