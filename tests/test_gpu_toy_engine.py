"""Toy models through the whole engine (scheduler, run-ahead, CUDA graphs), defined and registered here alone: a
mixer with state of its own per request that plans its captured steps itself and wants its prompts cut at multiples
of 8, and layers with a window beside layers without (two cache groups, pages given back while a request runs).
Each is compared with the same engine run step by step, without graphs and without a step in flight."""
from __future__ import annotations

import pytest
import torch

from holon_b200.config import LayerSpec, ModelSpec, PartRef, Run, WeightRule, register_architecture, unregister_architecture
from holon_b200.engine import Engine, EngineConfig, SamplingParams
from holon_b200.parts import Part, SlotState, register_part, unregister_part
from holon_b200.weights import RandomSource
from test_gpu_toy_parts import window_recipe

pytestmark = pytest.mark.gpu


class RunningMean(Part):
    """out_t = W · mean(x_0 .. x_t): the sum of the inputs and their count live in the request's slot. A step of
    one-token rows is all device work (it can be captured); rows of several tokens are walked on the host."""

    plans: list = []                                   # what capture_plan answered, step by step
    cuts: list = []                                    # (tokens before, tokens brought) of every row of several tokens

    def __init__(self, ctx, *, hidden, layer=0):
        super().__init__()
        self.ctx, self.hidden = ctx, hidden
        self.weight = self.add_param("weight", (hidden, hidden), "matrix")

    def cache(self):
        return None

    def slot_states(self):
        return (SlotState("sum", (self.hidden,), chunk=8), SlotState("count", (1,)))

    def capture_plan(self, step, max_model_len):
        """A plan of its own: a graph per 16 tokens of the longest row (it stands for any host-side decision that a
        captured launch freezes)."""
        answer = ("running_mean", int(step.rows.host_kv_len.max()) // 16)
        RunningMean.plans.append(answer)
        return answer

    def forward(self, x, step, cache):
        rows, out = step.rows, torch.empty_like(x)
        if rows.n_tokens == rows.n_rows:                                   # one token a row: no host work
            slots = rows.row_slot.long()
            sums = cache.slots["sum"][slots] + x.float()
            counts = cache.slots["count"][slots] + 1
            cache.slots["sum"][slots] = sums
            cache.slots["count"][slots] = counts
            self.ctx.kernels.linear(out, (sums / counts).to(x.dtype).contiguous(), self.weight.tensor)
            return out
        qs, lens = rows.host_query_start, rows.host_kv_len
        for b, slot in enumerate(rows.row_slot.tolist()):
            a, e = int(qs[b]), int(qs[b + 1])
            if e - a > 1:
                RunningMean.cuts.append((int(lens[b]) - (e - a), e - a))
            piece = x[a:e].float()
            sums = cache.slots["sum"][slot] + piece.cumsum(0)
            counts = cache.slots["count"][slot] + torch.arange(1, e - a + 1, device=x.device)[:, None]
            self.ctx.kernels.linear(out[a:e], (sums / counts).to(x.dtype).contiguous(), self.weight.tensor)
            cache.slots["sum"][slot] = sums[-1]
            cache.slots["count"][slot] = counts[-1]
        return out


def mean_recipe(c):
    norm = PartRef.of("norm", "rmsnorm", eps=1e-6)
    attention = PartRef.of("mixer", "gqa", heads=4, kv_heads=2, head_dim=16, qk_norm=norm, window=0,
                           position=PartRef.of("position", "rope", theta=1e4, rotary_dim=16))
    ffn = PartRef.of("ffn", "swiglu", inter=c["inter"])
    block = PartRef.of("block", "prenorm")
    layers = (LayerSpec(block, attention, ffn, norm), LayerSpec(block, PartRef.of("mixer", "toy_running_mean"), ffn, norm))
    return ModelSpec(hidden=c["hidden"], vocab=c["vocab"], layers=layers, order=(Run(0, 0), Run(1, 1)),
                     embed=PartRef.of("embed", "table"), norm=norm, head=PartRef.of("head", "linear", tied=False),
                     weight_rules=(WeightRule("{rest}", "{rest}"),))


def prompts_of(vocab, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


def generate(config, seed, prompts, max_tokens, **kw):
    args = dict(model="toy", dtype="float32", page_size=8, max_seqs=4, max_model_len=160, max_step_tokens=21,
                state_memory=8 << 20, seed=1)
    args.update(kw)
    engine = Engine(EngineConfig(**args), source=RandomSource(config, seed=seed, dtype=torch.float32))
    params = [SamplingParams(temperature=1.0, max_tokens=max_tokens, seed=70 + i) for i in range(len(prompts))]
    out = engine.generate(prompts, params)
    engine.built.cache.check()
    assert not engine.built.cache.live
    return engine, out


def test_a_mixer_with_state_of_its_own_through_run_ahead_and_graphs():
    """The state is updated once a step, also in the step that records a new graph while the step before is still in
    flight; the mixer's own answer to `capture_plan` keys the graphs; its prompts are cut at multiples of 8."""
    register_part("mixer", "toy_running_mean", RunningMean)
    register_architecture("ToyMeanEngineForCausalLM", dict, mean_recipe)
    try:
        config = {"architectures": ["ToyMeanEngineForCausalLM"], "hidden": 64, "vocab": 97, "inter": 80}
        prompts = prompts_of(97, (30, 13, 9, 3), 5)
        RunningMean.plans, RunningMean.cuts = [], []
        engine, got = generate(config, 3, prompts, 40)
        assert engine.built.cache.chunk == 8
        cuts = list(RunningMean.cuts)
        assert any(before > 0 for before, _ in cuts)                                   # prompts were cut
        for before, n in cuts:                                                          # ... only at multiples of 8
            assert (before + n) % 8 == 0 or any(before + n == len(p) for p in prompts), (before, n)
        keys = list(engine._graphs)
        toy_plans = {plan for key in keys for plan in key[3] if plan and plan[0] == "running_mean"}
        assert len(toy_plans) >= 3 and len(keys) >= 3                                  # a graph per answer of the mixer
        assert engine._captured_ahead                                                  # some recorded with a step in flight
        assert engine.stats()["graph_steps"] > 20
        _, want = generate(config, 3, prompts, 40, overlap=False, cuda_graphs=False)
        assert got == want and any(len(set(t)) > 5 for t in got)
    finally:
        unregister_part("mixer", "toy_running_mean")
        unregister_architecture("ToyMeanEngineForCausalLM")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_windowed_layers_through_run_ahead_and_graphs(dtype):
    """Layers with a window give pages back while their requests decode; the block-table rows that change travel with
    the step they belong to, so a step in flight never sees what the host did to the table for the next one."""
    register_architecture("ToyWindowEngineForCausalLM", dict, window_recipe)
    try:
        config = {"architectures": ["ToyWindowEngineForCausalLM"], "hidden": 64, "vocab": 113, "inter": 96, "head_dim": 16,
                  "window": 18}                                                         # window % page == 2
        prompts = prompts_of(113, (41, 7, 22, 3), 9)
        kw = dict(dtype=dtype, max_step_tokens=64, max_model_len=128)
        engine, got = generate(config, 13, prompts, 60, **kw)
        assert len(engine.built.cache.groups) == 2 and engine.stats()["graph_steps"] > 30
        _, in_turn = generate(config, 13, prompts, 60, overlap=False, **kw)             # same graphs, no step in flight
        assert got == in_turn
        if dtype == "float32":
            _, want = generate(config, 13, prompts, 60, overlap=False, cuda_graphs=False, **kw)
            assert got == want
        assert any(len(set(t)) > 5 for t in got)
    finally:
        unregister_architecture("ToyWindowEngineForCausalLM")


def test_prefix_cache_with_windowed_layers_on_the_device():
    """Two cache groups, one with a window, and prompts with an equal beginning, twice over, under run-ahead and graphs:
    requests start in the middle of their prompts in both groups (in the windowed one on the pages that reach into the
    window only) and generate what an engine without the prefix cache generates."""
    register_architecture("ToyWindowPrefixEngineForCausalLM", dict, window_recipe)
    try:
        config = {"architectures": ["ToyWindowPrefixEngineForCausalLM"], "hidden": 64, "vocab": 113, "inter": 96,
                  "head_dim": 16, "window": 18}
        stem = prompts_of(113, (50,), 4)[0]
        prompts = [stem + tail for tail in prompts_of(113, (1, 9, 20), 6)] + [stem[:27], stem]

        def run(**kw):
            args = dict(model="toy", dtype="float32", page_size=8, max_seqs=4, max_model_len=128, max_step_tokens=32,
                        chunk_with_decode=8, state_memory=8 << 20, seed=1)
            args.update(kw)
            engine = Engine(EngineConfig(**args), source=RandomSource(config, seed=13, dtype=torch.float32))
            params = [SamplingParams(temperature=1.0, max_tokens=24, seed=30 + i) for i in range(len(prompts))]
            out = [engine.generate(prompts, params) for _ in range(2)]
            engine.built.cache.check()
            assert not engine.built.cache.live
            return engine, out

        engine, got = run()
        prefix = engine.built.cache.prefix
        assert prefix is not None and sorted(prefix.windows) == [0, 18]
        assert engine.stats()["prefix_hit_tokens"] >= 5 * 24 and engine.stats()["graph_steps"] > 20
        _, want = run(prefix_cache=False)
        assert got == want and got[0] == got[1] and any(len(set(t)) > 3 for t in got[0])
    finally:
        unregister_architecture("ToyWindowPrefixEngineForCausalLM")
