"""Two more toy parts that are defined here, registered, built into a model and stepped without any change to the
framework: a feed-forward that routes every token to one of several experts, and a position encoding whose angles
grow with the logarithm of the position. The model that holds them is compared, whole and in portions, with the
formulas written out below; it is nobody's architecture. A second toy model puts layers with a window beside layers
without one (two cache groups)."""
from __future__ import annotations

import pytest
import torch

import plain_qwen3 as plain
from holon_b200.config import LayerSpec, ModelSpec, PartRef, Run, WeightRule, register_architecture, unregister_architecture
from holon_b200.engine import StepEntry, build
from holon_b200.parts import Part, register_part, unregister_part
from holon_b200.weights import RandomSource

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HEADS, KV_HEADS, HEAD_DIM, EXPERTS, EXPERT_INTER, EPS = 6, 3, 16, 5, 40, 1e-5


class TopOneExperts(Part):
    """out = p_e · W2_e · relu(W1_e · x) for the expert e with the largest router logit, p = softmax(logits) in
    32-bit. Tokens are sorted by expert on the device, so no step's shape depends on where they went."""

    def __init__(self, ctx, *, experts, inter, hidden, layer=0):
        super().__init__()
        self.ctx, self.experts, self.inter, self.hidden = ctx, experts, inter, hidden
        self.router = self.add_param("router", (experts, hidden), "matrix")
        self.w1 = self.add_param("w1", (experts * inter, hidden), "matrix")
        self.w2 = self.add_param("w2", (experts * hidden, inter), "matrix")

    def forward(self, x, step):
        k, t = self.ctx.kernels, x.shape[0]
        logits = torch.empty(t, self.experts, dtype=x.dtype, device=x.device)
        k.linear(logits, x, self.router.tensor)
        prob, choice = torch.softmax(logits.float(), dim=-1).max(dim=-1)
        out = torch.zeros_like(x)
        for e in range(self.experts):
            rows = (choice == e).nonzero().flatten()
            if rows.numel() == 0:
                continue
            xe = x[rows].contiguous()
            hidden = torch.empty(rows.numel(), self.inter, dtype=x.dtype, device=x.device)
            k.linear(hidden, xe, self.w1.tensor[e * self.inter:(e + 1) * self.inter])
            ye = torch.empty(rows.numel(), self.hidden, dtype=x.dtype, device=x.device)
            k.linear(ye, torch.relu(hidden), self.w2.tensor[e * self.hidden:(e + 1) * self.hidden])
            out[rows] = (ye.float() * prob[rows, None]).to(x.dtype)
        return out


class LogRotation(Part):
    """angle_i(p) = log(1 + p) · base^(−2i/rotary_dim): the same interface as the built-in rotation (a table of
    cosines then sines per position, and `rotary_dim`), other angles."""

    def __init__(self, ctx, *, base, rotary_dim, head_dim):
        super().__init__()
        self.base, self.rotary_dim = float(base), rotary_dim
        self.table = self.angles(ctx.max_positions).to(ctx.device)

    def angles(self, positions):
        rd = self.rotary_dim
        inv_freq = 1.0 / (self.base ** (torch.arange(0, rd, 2, dtype=torch.float32) / rd))
        angle = torch.log1p(torch.arange(positions, dtype=torch.float32))[:, None] * inv_freq[None, :]
        return torch.cat((angle.cos(), angle.sin()), dim=-1).contiguous()


def toy_recipe(c):
    norm = PartRef.of("norm", "rmsnorm", eps=EPS)
    log_attention = PartRef.of("mixer", "gqa", heads=HEADS, kv_heads=KV_HEADS, head_dim=HEAD_DIM, qk_norm=norm, window=0,
                               position=PartRef.of("position", "toy_log", base=50.0, rotary_dim=8))
    attention = PartRef.of("mixer", "gqa", heads=HEADS, kv_heads=KV_HEADS, head_dim=HEAD_DIM, qk_norm=norm, window=0,
                           position=PartRef.of("position", "rope", theta=1e4, rotary_dim=HEAD_DIM))
    routed = PartRef.of("ffn", "toy_top_one", experts=EXPERTS, inter=EXPERT_INTER)
    block = PartRef.of("block", "prenorm")
    layers = (LayerSpec(block, log_attention, routed, norm),
              LayerSpec(block, attention, PartRef.of("ffn", "swiglu", inter=c["inter"]), norm),
              LayerSpec(block, log_attention, routed, norm))
    return ModelSpec(hidden=c["hidden"], vocab=c["vocab"], layers=layers, order=tuple(Run(i, i) for i in range(3)),
                     embed=PartRef.of("embed", "table"), norm=norm, head=PartRef.of("head", "linear", tied=False),
                     weight_rules=(WeightRule("{rest}", "{rest}"),))


# ---------------------------------------------------------------- the same model written out, whole sequences, no cache

def rotate(x, table, rotary_dim):
    """Half-split pairs (i, i + rotary_dim / 2) of the first rotary_dim dimensions; the rest passes through."""
    half = rotary_dim // 2
    cos, sin = table[: x.shape[0], None, :half], table[: x.shape[0], None, half:]
    a, b = x[..., :half], x[..., half:rotary_dim]
    return torch.cat((a * cos - b * sin, b * cos + a * sin, x[..., rotary_dim:]), dim=-1)


def plain_attention(x, mixer):
    t, heads, kv_heads, d = x.shape[0], mixer.heads, mixer.kv_heads, mixer.head_dim
    w = mixer.qkv.weight.tensor.float().cpu()
    q, k, v = (x @ w.T).split((heads * d, kv_heads * d, kv_heads * d), dim=-1)
    q = plain.rms_norm(q.reshape(t, heads, d), mixer.q_norm.weight.tensor.float().cpu(), EPS)
    k = plain.rms_norm(k.reshape(t, kv_heads, d), mixer.k_norm.weight.tensor.float().cpu(), EPS)
    table, rd = mixer.position.table.cpu(), mixer.position.rotary_dim
    o = plain.causal_attention(rotate(q, table, rd), rotate(k, table, rd), v.reshape(t, kv_heads, d), mixer.window)
    return o.reshape(t, heads * d) @ mixer.o_proj.weight.tensor.float().cpu().T


def plain_ffn(x, ffn):
    if not isinstance(ffn, TopOneExperts):
        gate, up = (x @ ffn.gate_up.weight.tensor.float().cpu().T).chunk(2, dim=-1)
        return (torch.nn.functional.silu(gate) * up) @ ffn.down.weight.tensor.float().cpu().T
    prob, choice = torch.softmax(x @ ffn.router.tensor.float().cpu().T, dim=-1).max(dim=-1)
    w1 = ffn.w1.tensor.float().cpu().view(EXPERTS, EXPERT_INTER, -1)
    w2 = ffn.w2.tensor.float().cpu().view(EXPERTS, -1, EXPERT_INTER)
    rows = [prob[i] * (w2[choice[i]] @ torch.relu(w1[choice[i]] @ x[i])) for i in range(x.shape[0])]
    return torch.stack(rows), choice


def plain_forward(model, ids):
    h = plain.embedding(ids, model.embed.weight.tensor.float().cpu())
    choices = []
    for block in model.layers:
        h = h + plain_attention(plain.rms_norm(h, block.input_norm.weight.tensor.float().cpu(), EPS), block.mixer)
        y = plain_ffn(plain.rms_norm(h, block.post_norm.weight.tensor.float().cpu(), EPS), block.ffn)
        if isinstance(y, tuple):
            y, choice = y
            choices.append(choice)
        h = h + y
    h = plain.rms_norm(h, model.norm.weight.tensor.float().cpu(), EPS)
    head = model.head.weight if model.head.weight is not None else model.embed.weight        # a tied head reads the table
    return h @ head.tensor.float().cpu().T, choices


def test_toy_routed_feed_forward_and_toy_position_encoding():
    register_part("ffn", "toy_top_one", TopOneExperts)
    register_part("position", "toy_log", LogRotation)
    register_architecture("ToyRoutedForCausalLM", dict, toy_recipe)
    try:
        config = {"architectures": ["ToyRoutedForCausalLM"], "hidden": 72, "vocab": 131, "inter": 56}
        b = build(RandomSource(config, seed=11, dtype=torch.float32), dtype="float32", device=DEV, page_size=8,
                  max_seqs=3, max_model_len=64, max_step_tokens=64, pages=14)
        g = torch.Generator().manual_seed(4)
        ids = torch.randint(0, 131, (37,), generator=g).tolist()
        other = torch.randint(0, 131, (9,), generator=g).tolist()
        want, choices = plain_forward(b.model, ids)
        assert all(len(set(c.tolist())) >= 3 for c in choices)           # the router does send tokens to several experts

        def run(portions, beside=False):
            slot, at, rows = b.cache.admit(), 0, []
            extra = b.cache.admit() if beside else None
            for i, n in enumerate(portions):
                b.cache.reserve(slot, at + n)
                entries = [StepEntry(slot, ids[at:at + n], at, range(n))]
                if beside and i < len(other):                            # another request decodes in the same steps
                    b.cache.reserve(extra, i + 1)
                    entries.insert(0, StepEntry(extra, other[i:i + 1], i))
                rows.append(b.runner.step(entries))
                at += n
            b.cache.release(slot)
            if beside:
                b.cache.release(extra)
            return torch.cat(rows).cpu()

        for portions, beside in (([37], False), ([20] + [1] * 17, False), ([2, 9, 3, 16, 7], False), ([5, 2, 11, 4, 15], True)):
            got = run(portions, beside)
            assert (got - want).abs().max() < 1e-4, (portions, float((got - want).abs().max()))
            assert torch.equal(got.argmax(-1), want.argmax(-1))
    finally:
        unregister_part("ffn", "toy_top_one")
        unregister_part("position", "toy_log")
        unregister_architecture("ToyRoutedForCausalLM")


# ---------------------------------------------------------------- layers with a window beside layers without: two cache groups

def window_recipe(c):
    norm = PartRef.of("norm", "rmsnorm", eps=EPS)
    rope = PartRef.of("position", "rope", theta=1e4, rotary_dim=c["head_dim"])
    full = PartRef.of("mixer", "gqa", heads=4, kv_heads=2, head_dim=c["head_dim"], qk_norm=norm, window=0, position=rope)
    near = PartRef.of("mixer", "gqa", heads=4, kv_heads=2, head_dim=c["head_dim"], qk_norm=norm, window=c["window"], position=rope)
    ffn = PartRef.of("ffn", "swiglu", inter=c["inter"])
    block = PartRef.of("block", "prenorm")
    layers = tuple(LayerSpec(block, mixer, ffn, norm) for mixer in (near, full, near, full))
    return ModelSpec(hidden=c["hidden"], vocab=c["vocab"], layers=layers, order=tuple(Run(i, i) for i in range(4)),
                     embed=PartRef.of("embed", "table"), norm=norm, head=PartRef.of("head", "linear", tied=True),
                     weight_rules=(WeightRule("{rest}", "{rest}"),))


@pytest.mark.parametrize("dtype,head_dim,page,window,tol", [("float32", 16, 8, 20, 1e-4), ("bfloat16", 16, 8, 20, 6e-2),
                                                            ("bfloat16", 128, 64, 150, 6e-2)])
def test_layers_with_a_window_beside_layers_without(dtype, head_dim, page, window, tol):
    """Two layers that see only the last `window` keys and two that see all: two cache groups with pools and block
    tables of their own. Whole, in portions and token by token give the plain formula's logits, and in the window's group
    a request never holds more pages than its window and the step's portion span: the pages it has passed come back
    (head size 128 with pages of 64 puts the prompt portions on the tcgen05 kernel)."""
    register_architecture("ToyWindowForCausalLM", dict, window_recipe)
    try:
        config = {"architectures": ["ToyWindowForCausalLM"], "hidden": 64, "vocab": 113, "inter": 96, "head_dim": head_dim,
                  "window": window}
        n = 5 * window // 2 + 7
        b = build(RandomSource(config, seed=13, dtype=torch.float32), dtype=dtype, device=DEV, page_size=page, max_seqs=2,
                  max_model_len=-(-(n + 8) // page) * page, max_step_tokens=512, pages=-(-n // page) + 3)
        assert len(b.cache.groups) == 2
        near = next(g for g in b.cache.groups if g.decl.window)
        ids = torch.randint(0, 113, (n,), generator=torch.Generator().manual_seed(6)).tolist()
        want, _ = plain_forward(b.model, ids)

        def run(portions):
            slot, at, rows, held = b.cache.admit(), 0, [], 0
            for size in portions:
                b.cache.reserve(slot, at + size)
                rows.append(b.runner.step([StepEntry(slot, ids[at:at + size], at, range(size))]))
                at += size
                held = max(held, int((near.table[slot] != near.null_page).sum()))
            b.cache.release(slot)
            b.cache.check()
            return torch.cat(rows).float().cpu(), held

        for portions in ([n], [window + 3, 2, n - window - 5 - 9] + [1] * 9, [7] * (n // 7) + [n % 7] * (1 if n % 7 else 0)):
            got, held = run(portions)
            diff = float((got - want).abs().max())
            assert diff < tol, (portions[:4], diff)
            if len(portions) > 1:
                assert held <= -(-window // page) + -(-max(portions) // page) + 1      # never the whole sequence's pages
    finally:
        unregister_architecture("ToyWindowForCausalLM")
