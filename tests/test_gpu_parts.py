"""Each part alone on the GPU against the plain implementation's function for it, and a toy mixer with state of its
own that is defined here, registered, built into a model and stepped without any change to the framework."""
from __future__ import annotations


import pytest
import torch

import plain_qwen3 as plain
from holon_b200.cache import CacheManager
from holon_b200.config import LayerSpec, ModelSpec, PartRef, Run, WeightRule, register_architecture, unregister_architecture
from holon_b200.engine import StepEntry, build
from holon_b200.engine.runner import Runner
from holon_b200.parts import BuildContext, CacheEntry, Part, Residual, SlotState, register_part, unregister_part
from holon_b200.weights import RandomSource

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = {"float32": (torch.float32, 2e-5), "bfloat16": (torch.bfloat16, 2e-2)}


def ctx_of(dtype, max_positions=256):
    from holon_b200.kernels import load_kernels
    return BuildContext(DEV, dtype, load_kernels(DEV), max_positions=max_positions, max_step_tokens=256)


def fill(part, seed, dtype):
    """Seeded values for every parameter of a part; returns them as float32 CPU tensors by loadable name."""
    g, named = torch.Generator().manual_seed(seed), {}
    for _, p in part.params():
        value = torch.randn(p.shape, generator=g) * (0.1 if p.kind == "gain" else 0.08) + (1.0 if p.kind == "gain" else 0.0)
        p.tensor = value.to(dtype).to(DEV)
    for name, p, (a, b) in part.loadables():
        named[name] = p.tensor[a:b].float().cpu()
    return named


def close(got, want, tol, scale=1.0):
    diff = float((got.float().cpu() - want).abs().max())
    assert diff <= tol * scale, f"difference {diff}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm(dtype):
    dt, tol = DTYPES[dtype]
    norm = ctx_of(dt).part(PartRef.of("norm", "rmsnorm", eps=1e-5), dim=200)
    w = fill(norm, 1, dt)["weight"]
    h = torch.randn(9, 200, generator=torch.Generator().manual_seed(2))
    delta = torch.randn(9, 200, generator=torch.Generator().manual_seed(3)).to(dt)
    stream = Residual(h.to(DEV), delta.to(DEV))
    picked = norm.gather(stream, torch.tensor([8, 2], dtype=torch.int32, device=DEV))
    close(picked, plain.rms_norm(h + delta.float(), w, 1e-5)[[8, 2]], tol, 4)
    out = norm.add(stream)
    close(out, plain.rms_norm(h + delta.float(), w, 1e-5), tol, 4)
    assert stream.delta is None and torch.allclose(stream.h.cpu(), h + delta.float(), atol=1e-6)
    close(norm.apply(delta.to(DEV)), plain.rms_norm(delta.float(), w, 1e-5), tol, 4)


def test_rope_table():
    rope = ctx_of(torch.float32).part(PartRef.of("position", "rope", theta=5e5, rotary_dim=48), head_dim=48)
    x = torch.randn(7, 3, 48, generator=torch.Generator().manual_seed(4))
    positions = torch.tensor([0, 1, 5, 100, 255, 31, 32])
    table = rope.table.cpu()[positions]
    cos, sin = table[:, None, :24], table[:, None, 24:]
    mine = torch.cat((x[..., :24] * cos - x[..., 24:] * sin, x[..., 24:] * cos + x[..., :24] * sin), -1)
    assert (mine - plain.rope(x, positions, 5e5)).abs().max() < 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_and_embedding_and_head(dtype):
    dt, tol = DTYPES[dtype]
    ctx = ctx_of(dt)
    ffn = ctx.part(PartRef.of("ffn", "swiglu", inter=176), hidden=96, layer=0)
    w = fill(ffn, 5, dt)
    x = (torch.randn(11, 96, generator=torch.Generator().manual_seed(6))).to(dt)
    close(ffn.forward(x.to(DEV), None), plain.swiglu(x.float(), w, ""), tol, 2)
    embed = ctx.part(PartRef.of("embed", "table"), vocab=389, hidden=96)
    table = fill(embed, 7, dt)["weight"]
    ids = torch.tensor([0, 388, 17], dtype=torch.int32)
    assert torch.equal(embed.forward(ids.to(DEV)).h.cpu(), table[ids.long()])
    for tied in (True, False):
        head = ctx.part(PartRef.of("head", "linear", tied=tied), vocab=389, hidden=96, embed=embed)
        hw = table if tied else fill(head, 8, dt)["weight"]
        logits = head.forward(x.to(DEV))
        assert logits.dtype == torch.float32
        close(logits, x.float() @ hw.T, tol, 2)


def one_sequence(ctx, mixer_like, n, page_size=8):
    """A cache and a step context for one request of n tokens, all new."""
    entries = [CacheEntry(0, 0, mixer_like.cache(), tuple(mixer_like.slot_states()))]
    cache = CacheManager(entries, page_size, 2, 256, ctx.dtype, DEV, pages=40)

    class OneLayer:                                   # the least a Runner needs of a model
        spec = type("S", (), {"vocab": 10})
    runner = Runner(OneLayer, cache, ctx, 256)
    slot = cache.admit()
    cache.reserve(slot, n)
    step = runner.context([StepEntry(slot, [0] * n, 0)])
    return step, step.layer_cache(Run(0, 0))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [0, 5])
def test_attention_and_block(dtype, window):
    dt, tol = DTYPES[dtype]
    ctx = ctx_of(dt)
    config = dict(num_attention_heads=6, num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-5, rope_theta=1e4)
    norm = PartRef.of("norm", "rmsnorm", eps=1e-5)
    mixer_ref = PartRef.of("mixer", "gqa", heads=6, kv_heads=2, head_dim=32, qk_norm=norm, window=window,
                           position=PartRef.of("position", "rope", theta=1e4, rotary_dim=32))
    mixer = ctx.part(mixer_ref, hidden=96, layer=0)
    w = fill(mixer, 9, dt)
    n = 29
    x = torch.randn(n, 96, generator=torch.Generator().manual_seed(10)).to(dt)
    step, cache = one_sequence(ctx, mixer, n)
    got = mixer.forward(x.to(DEV), step, cache)
    want = plain.attention_layer(x.float(), w, "", config, torch.arange(n), window)
    close(got, want, tol, 2)
    if window:
        return
    block = ctx.part(PartRef.of("block", "prenorm"), layer=0, hidden=96, mixer=mixer_ref,
                     ffn=PartRef.of("ffn", "swiglu", inter=160), norm=norm)
    w = fill(block, 11, dt)
    names = {"input_norm.": "model.layers.0.input_layernorm.", "post_norm.": "model.layers.0.post_attention_layernorm.",
             "mixer.": "model.layers.0.self_attn.", "ffn.": "model.layers.0.mlp."}
    stored = {next(v + k[len(p):] for p, v in names.items() if k.startswith(p)): t for k, t in w.items()}
    h = torch.randn(n, 96, generator=torch.Generator().manual_seed(12))
    step, cache = one_sequence(ctx, block.mixer, n)
    stream = block.forward(Residual(h.to(DEV)), step, cache)
    got = stream.h.cpu() + stream.delta.float().cpu()                  # the feed-forward's output is still pending
    want = plain.block(h, stored, 0, dict(config, hidden_size=96), torch.arange(n))
    close(got, want, tol, 4)


# ---------------------------------------------------------------- a toy mixer with state of its own

class RunningMean(Part):
    """out_t = W · mean(x_0 .. x_t): the sum of the inputs and their count live in the request's slot."""

    def __init__(self, ctx, *, hidden, layer=0):
        super().__init__()
        self.ctx, self.hidden = ctx, hidden
        self.weight = self.add_param("weight", (hidden, hidden), "matrix")

    def cache(self):
        return None                                    # no pages

    def slot_states(self):
        return (SlotState("sum", (self.hidden,)), SlotState("count", (1,)))

    def forward(self, x, step, cache):
        out = torch.empty_like(x)
        qs, slots = step.rows.host_query_start, step.rows.row_slot.tolist()
        for b, slot in enumerate(slots):
            rows = x[int(qs[b]):int(qs[b + 1])].float()
            sums = cache.slots["sum"][slot] + rows.cumsum(0)
            counts = cache.slots["count"][slot] + torch.arange(1, rows.shape[0] + 1, device=x.device)[:, None]
            mean = (sums / counts).to(x.dtype)
            self.ctx.kernels.linear(out[int(qs[b]):int(qs[b + 1])], mean.contiguous(), self.weight.tensor)
            cache.slots["sum"][slot] = sums[-1]
            cache.slots["count"][slot] = counts[-1]
        return out


def toy_recipe(c):
    norm = PartRef.of("norm", "rmsnorm", eps=1e-6)
    attention = PartRef.of("mixer", "gqa", heads=4, kv_heads=2, head_dim=16, qk_norm=norm, window=0,
                           position=PartRef.of("position", "rope", theta=1e4, rotary_dim=16))
    ffn = PartRef.of("ffn", "swiglu", inter=c["inter"])
    block = PartRef.of("block", "prenorm")
    layers = (LayerSpec(block, attention, ffn, norm), LayerSpec(block, PartRef.of("mixer", "running_mean"), ffn, norm))
    # layer 0 runs three times: filling entry 0, filling entry 2, and once more reading entry 0 without writing it
    order = (Run(0, 0), Run(1, 1), Run(0, 2), Run(0, 0, fills=False))
    return ModelSpec(hidden=c["hidden"], vocab=c["vocab"], layers=layers, order=order,
                     embed=PartRef.of("embed", "table"), norm=norm, head=PartRef.of("head", "linear", tied=True),
                     weight_rules=(WeightRule("{rest}", "{rest}"),))


def test_toy_mixer_with_state_is_registered_built_and_stepped():
    register_part("mixer", "running_mean", RunningMean)
    register_architecture("ToyMeanForCausalLM", dict, toy_recipe)
    try:
        config = {"architectures": ["ToyMeanForCausalLM"], "hidden": 64, "vocab": 97, "inter": 80}
        b = build(RandomSource(config, seed=3, dtype=torch.float32), dtype="float32", device=DEV, page_size=8,
                  max_seqs=3, max_model_len=64, max_step_tokens=64, pages=12)
        assert [e.decl is None for e in b.model.entries] == [False, True, False]        # layer 0 fills two entries
        assert set(b.cache.slot_states) == {(1, "sum"), (1, "count")}
        ids = [5, 96, 33, 0, 17, 42, 8, 8, 61, 2, 77]
        other = [9, 1, 4]

        def run(portions, beside=False):
            slot, at, rows = b.cache.admit(), 0, []
            extra = b.cache.admit() if beside else None
            for i, n in enumerate(portions):
                b.cache.reserve(slot, at + n)
                entries = [StepEntry(slot, ids[at:at + n], at, range(n))]
                if beside and i < len(other):                                       # another request in the same steps
                    b.cache.reserve(extra, i + 1)
                    entries.insert(0, StepEntry(extra, other[i:i + 1], i))
                rows.append(b.runner.step(entries))
                at += n
            b.cache.release(slot)
            if beside:
                b.cache.release(extra)
            return torch.cat(rows).cpu()

        whole = run([len(ids)])
        assert whole.shape == (len(ids), 97) and torch.isfinite(whole).all()
        assert (run([4, 2, 5]) - whole).abs().max() < 1e-4                         # state carries across steps
        assert (run([1] * len(ids)) - whole).abs().max() < 1e-4
        assert (run([3, 1, 1, 6], beside=True) - whole).abs().max() < 1e-4          # and is kept apart per request
        # the toy layer alone against its formula
        mixer = b.model.layers[1].mixer
        x = torch.randn(6, 64, generator=torch.Generator().manual_seed(1))
        slot = b.cache.admit()
        b.cache.reserve(slot, 6)
        step = b.runner.context([StepEntry(slot, [0] * 6, 0)])
        got = mixer.forward(x.to(DEV), step, step.layer_cache(Run(1, 1))).cpu()
        want = (x.cumsum(0) / torch.arange(1, 7)[:, None]) @ mixer.weight.tensor.cpu().T
        assert (got - want).abs().max() < 1e-5
    finally:
        unregister_part("mixer", "running_mean")
        unregister_architecture("ToyMeanForCausalLM")
