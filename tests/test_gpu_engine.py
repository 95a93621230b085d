"""Generation through the public entry point on the GPU (`Engine.generate`, host token ids in and out) against the
plain implementation: greedy and seeded temperature sampling, with prompt portions beside decoding requests, with
CUDA graphs on and off, and in a pool so small that requests are preempted and computed again."""
from __future__ import annotations

import dataclasses

import pytest

import plain_qwen3 as plain
from helpers import make_folder, random_prompt
from holon_b200.engine import Engine, EngineConfig, SamplingParams

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=["a", "b", "c"])
def model(request, tmp_path_factory):
    folder = make_folder(tmp_path_factory.mktemp("models"), request.param)
    config, weights = plain.read_folder(folder)
    prompts = [random_prompt(config["vocab_size"], n, 60 + n) for n in (5, 17, 31, 1, 40, 77)]
    return folder, config, weights, prompts


def engine_of(folder, dtype, **kw):
    args = dict(model=str(folder), dtype=dtype, page_size=16, max_seqs=4, max_model_len=128, max_step_tokens=48,
                chunk_with_decode=8, state_memory=4 << 20, seed=3)
    args.update(kw)
    return Engine(EngineConfig(**args))


def check_teacher_forced(config, weights, prompt, tokens, params, seed, exact):
    """Every generated token against the plain implementation's logits at its place. float32: the very token.
    bfloat16: greedy tokens must be within a small margin of the best logit (a near-tie may flip)."""
    ids = list(prompt)
    for token in tokens:
        logits = plain.forward(config, weights, ids)[-1]
        if exact:
            want = plain.sample(logits, params.temperature, seed, len(ids), params.top_k, params.top_p, params.min_p)
            assert token == want, (len(ids), token, want)
        else:
            assert float(logits[token]) >= float(logits.max()) - 0.06
        ids.append(token)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("graphs", [True, False])
def test_greedy_generation(model, dtype, graphs):
    folder, config, weights, prompts = model
    engine = engine_of(folder, dtype, cuda_graphs=graphs)
    params = SamplingParams(temperature=0.0, max_tokens=12)
    got = engine.generate(prompts, params)
    assert [len(g) for g in got] == [12] * len(prompts)
    for prompt, tokens in zip(prompts, got):
        check_teacher_forced(config, weights, prompt, tokens, params, 0, exact=dtype == "float32")
    stats = engine.stats()
    assert stats["mixed_steps"] > 0 and (stats["graph_steps"] > 0) == graphs
    assert (stats["mixed_graph_steps"] > 0) == graphs          # prompt portions that fill the budget beside decode rows
    engine.built.cache.check()
    assert not engine.built.cache.live
    if dtype == "float32":
        again = engine_of(folder, dtype, cuda_graphs=not graphs, chunk_with_decode=0, max_step_tokens=128, page_size=4,
                          overlap=False)
        assert again.generate(prompts, params) == got            # other batching, other pages, depth 0: the same tokens


def test_the_sequences_of_one_request_stream_under_their_indices(model):
    """`n` = 3: three sequences under one id, each the same as a request of its own with that sequence's seed; the
    whole-prompt call refuses n > 1 (core/holon/core/engine.py:331-376, 473-477)."""
    from holon_b200.sampling.params import sequence_seed
    folder, config, weights, prompts = model
    engine = engine_of(folder, "bfloat16")
    params = SamplingParams(temperature=0.9, max_tokens=6, seed=41, n=3)
    rid = engine.add([3, 1, 4, 1, 5], params, rid="pi")
    got = {i: [] for i in range(3)}
    ended = set()
    while engine.has_work():
        for d in engine.step():
            assert d.rid == rid == "pi" and d.index not in ended
            got[d.index].extend(d.token_ids)
            if d.finish_reason:
                ended.add(d.index)
    assert ended == {0, 1, 2} and "pi" not in engine.requests and not engine.built.cache.live
    alone = [engine.generate([[3, 1, 4, 1, 5]], SamplingParams(temperature=0.9, max_tokens=6,
                                                               seed=sequence_seed(41, i)))[0] for i in range(3)]
    assert [got[i] for i in range(3)] == alone and len({tuple(a) for a in alone}) > 1
    with pytest.raises(ValueError, match="one sequence per prompt"):
        engine.generate([[1, 2]], params)
    engine.add([1, 2, 3], params, rid="gone")
    engine.step()
    assert sorted(d.index for d in engine.abort("gone")) == [0, 1, 2]
    engine.drain()
    assert not engine.has_work() and not engine.built.cache.live
    engine.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_logprobs_beside_requests_that_ask_for_none(model, dtype):
    """Generated-token and prompt logprobs through the CUDA kernels: steps that owe them run outside the graphs and
    give the tokens the same requests get without them; values against the plain implementation."""
    folder, config, weights, prompts = model
    engine = engine_of(folder, dtype)
    base = [SamplingParams(temperature=0.0, max_tokens=6) for _ in prompts]
    plain_tokens = engine.generate(prompts, base)
    asked = [dataclasses.replace(p, logprobs=(4, None, 0)[i % 3], prompt_logprobs=(None, 3)[i % 2]) for i, p in enumerate(base)]
    rids = [engine.add(p, sp) for p, sp in zip(prompts, asked)]
    seen = {rid: [] for rid in rids}
    while engine.has_work():
        for d in engine.step():
            seen[d.rid].append(d)
    tol = 1e-4 if dtype == "float32" else 0.08
    for rid, prompt, sp, want in zip(rids, prompts, asked, plain_tokens):
        deltas = seen[rid]
        if dtype == "float32":
            assert [t for d in deltas for t in d.token_ids] == want
        else:                                                      # (another batch shape may flip a near-tie in bfloat16)
            check_teacher_forced(config, weights, prompt, [t for d in deltas for t in d.token_ids], sp, 0, exact=False)
        first = deltas[0].prompt_logprobs
        if sp.prompt_logprobs is None:
            assert first is None
        else:
            whole = plain.forward(config, weights, list(prompt))
            assert len(first.token) == len(prompt) - 1
            for at in range(0, len(prompt) - 1, 5):
                own, _, top = plain.logprobs(whole[at], prompt[at + 1], sp.prompt_logprobs)
                assert abs(first.token[at] - own) < tol and len(first.top_ids[at]) == sp.prompt_logprobs
                assert all(abs(a - b) < tol for a, b in zip(first.top[at], top))
        ids = list(prompt)
        for d in deltas:
            if sp.logprobs is None:
                assert d.logprobs is None
            else:
                own, _, top = plain.logprobs(plain.forward(config, weights, ids)[-1], d.token_ids[0], sp.logprobs)
                assert abs(d.logprobs.token[0] - own) < tol and len(d.logprobs.top[0]) == sp.logprobs
                assert all(abs(a - b) < tol for a, b in zip(d.logprobs.top[0], top))
            ids += d.token_ids
    assert not engine._prompt_lp and not engine.built.cache.live
    engine.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefix_cache_on_the_device(model, dtype):
    """Prompts with an equal beginning, twice over: requests start on pages that earlier ones filled (CUDA graphs and
    prompt portions beside decode rows included) and generate what an engine without the prefix cache generates."""
    folder, config, weights, _ = model
    stem = random_prompt(config["vocab_size"], 70, 3)
    prompts = [stem + random_prompt(config["vocab_size"], n, 90 + n) for n in (1, 9, 30)] + [stem[:33], stem]
    params = SamplingParams(temperature=0.0, max_tokens=8)
    engine = engine_of(folder, dtype)
    assert engine.built.cache.prefix is not None
    first, second = engine.generate(prompts, params), engine.generate(prompts, params)
    stats = engine.stats()
    assert stats["prefix_hit_tokens"] >= 5 * 64 and stats["mixed_graph_steps"] > 0
    engine.built.cache.check()
    without = engine_of(folder, dtype, prefix_cache=False).generate(prompts, params)
    if dtype == "float32":
        assert first == second == without
    else:                                                          # (another batch shape may flip a near-tie in bfloat16)
        for prompt, a, b in zip(prompts, first, second):
            check_teacher_forced(config, weights, prompt, a, params, 0, exact=False)
            check_teacher_forced(config, weights, prompt, b, params, 0, exact=False)


def test_sampled_generation_is_seeded_and_survives_preemption(model):
    folder, config, weights, prompts = model
    params = [SamplingParams(temperature=0.8, max_tokens=10, seed=100 + i, top_k=(0, 20)[i % 2], top_p=(1.0, 0.9)[i // 3],
                             min_p=(0.0, 0.01)[i % 3 == 0]) for i in range(len(prompts))]
    roomy = engine_of(folder, "float32")
    got = roomy.generate(prompts, params)
    for prompt, tokens, p in zip(prompts, got, params):
        check_teacher_forced(config, weights, prompt, tokens, p, p.seed, exact=True)
    pages = -(-96 // 16) + 1                                         # one longest request and one page more
    tight = Engine(EngineConfig(model=str(folder), dtype="float32", page_size=16, max_seqs=4, max_model_len=96,
                                max_step_tokens=48, chunk_with_decode=8, seed=3,
                                state_memory=page_bytes(config, 16, 4) * (pages + 1)))
    assert tight.generate(prompts, params) == got
    assert tight.stats()["preemptions"] > 0
    tight.built.cache.check()


def page_bytes(config, page_size, itemsize):
    return config["num_hidden_layers"] * 2 * config["num_key_value_heads"] * page_size * config["head_dim"] * itemsize


def test_limits_and_errors(model):
    folder, config, _, _ = model
    engine = engine_of(folder, "float32", max_model_len=32)
    with pytest.raises(ValueError, match="empty"):
        engine.add([])
    with pytest.raises(ValueError, match="max_model_len"):
        engine.add(list(range(32)))
    with pytest.raises(ValueError, match="vocabulary"):
        engine.add([config["vocab_size"]])
    with pytest.raises(NotImplementedError):
        engine.add([1], SamplingParams(repetition_penalty=1.1))
    with pytest.raises(ValueError, match="logprobs"):
        engine.add([1], SamplingParams(logprobs=-3))
    out = engine.generate([[1, 2, 3]], SamplingParams(temperature=0.0))          # no max_tokens: stops at max_model_len
    assert len(out[0]) == 32 - 3
    rid = engine.add([4, 5, 6], SamplingParams(temperature=0.0, max_tokens=50))
    engine.step()
    assert [(d.index, d.finish_reason) for d in engine.abort(rid)] == [(0, "abort")] and engine.abort(rid) == []
    engine.drain()                                                   # (its first step was still in flight)
    assert not engine.has_work() and not engine.built.cache.live
    stop = out[0][2]
    cut = engine.generate([[1, 2, 3]], SamplingParams(temperature=0.0, stop_token_ids=(stop,)))
    assert cut[0] == out[0][:out[0].index(stop) + 1]


def test_generation_with_the_tcgen05_gemm(model):
    """The same greedy generation with every bfloat16 product of more than 16 rows on the hand-written tcgen05 kernel
    (SwiGLU fused into the gate/up product) instead of the library's."""
    folder, config, weights, prompts = model
    params = SamplingParams(temperature=0.0, max_tokens=6)
    engine = engine_of(folder, "bfloat16", max_step_tokens=128, chunk_with_decode=64)
    kernels = engine.built.ctx.kernels
    before = kernels.gemm
    kernels.gemm = "tcgen05"
    try:
        got = engine.generate(prompts, params)
        assert kernels.tcgen05_status() == 0
    finally:
        kernels.gemm = before
    for prompt, tokens in zip(prompts, got):
        check_teacher_forced(config, weights, prompt, tokens, params, 0, exact=False)


@pytest.mark.parametrize("overlap", [True, False])
def test_stop_tokens_while_a_step_is_in_flight(model, overlap):
    """With a step in flight a stop token is seen one step late: the request ends where it should, the row that was
    already enqueued for it is dropped, its slot comes back, and the other requests do not notice."""
    folder, config, weights, prompts = model
    free = engine_of(folder, "float32", overlap=overlap)
    base = free.generate(prompts[:3], SamplingParams(temperature=0.0, max_tokens=14))
    stops = [(b[4],) for b in base]                                 # each request stops at its own fifth token
    engine = engine_of(folder, "float32", overlap=overlap)
    params = [SamplingParams(temperature=0.0, max_tokens=14, stop_token_ids=s) for s in stops]
    got = engine.generate(prompts[:3], params)
    for g, b, s in zip(got, base, stops):
        assert g == b[:b.index(s[0]) + 1]
    engine.built.cache.check()
    assert not engine.built.cache.live and not engine.has_work()


def test_one_long_request_among_short_ones_takes_the_balanced_decode_graph(tmp_path):
    """A batch with one row far longer than the rest decodes through a graph captured with the keys shared out evenly;
    alike rows keep the graph with equal cuts. Both give the tokens of a run without graphs."""
    folder = make_folder(tmp_path, "a")
    config, _ = plain.read_folder(folder)
    prompts = [random_prompt(config["vocab_size"], n, 7 + n) for n in (4200, 30, 12, 55, 9, 21, 40, 3, 17, 26, 33, 8)]
    params = SamplingParams(temperature=0.0, max_tokens=12)          # the short ones still decode when the long one starts to
    kw = dict(page_size=64, max_seqs=12, max_model_len=4608, max_step_tokens=1024, chunk_with_decode=64)
    engine = engine_of(folder, "bfloat16", **kw)
    got = engine.generate(prompts, params)
    assert "balanced" in modes_of(engine._graphs)
    short = engine.generate(prompts[1:], params)
    assert modes_of(engine._graphs) == {"balanced", "splits"}
    plain_run = engine_of(folder, "bfloat16", cuda_graphs=False, **kw)
    kernels = plain_run.built.ctx.kernels                            # (one kernel table per device: put the setting back)
    before, kernels.decode_attention = kernels.decode_attention, "splits"
    try:
        assert plain_run.generate(prompts, params) == got and got[1:] == short
    finally:
        kernels.decode_attention = before
    engine.built.cache.check()


def modes_of(keys):
    """How the decode rows' keys are shared out in the graphs of `keys`: a key is (bucket, prompt portions, prompt
    tokens, the mixers' plans), and the attention's plan is (mode, bucket of the longest row)."""
    return {plan[0] for key in keys for plan in key[3] if plan is not None and plan[0] is not None}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_graph_captured_while_a_step_is_in_flight_runs_that_step_once(tmp_path, dtype):
    """In steady decode the host runs one step ahead: rows take their input token from the device. When the rows'
    lengths then call for another graph (the longest row passes 4,096 tokens beside short ones: the keys are shared
    out evenly from there on; short rows pass 512 tokens: the launch is planned for the next bucket), the first step
    of the new shape runs eagerly and is recorded, and must run once only: a replay on top would feed on the token the
    eager run has just stored. Tokens are sampled, so that a step that ran twice shows; they must equal those of an
    engine that commits every step before the next (same graphs, same plans: bit for bit), and in float32 those of
    an engine without graphs."""
    folder = make_folder(tmp_path, "b")
    config, _ = plain.read_folder(folder)
    vocab = config["vocab_size"]
    long_batch = [random_prompt(vocab, n, 7 + n) for n in (4088, 30, 12, 55, 9, 21, 40, 3, 17, 26, 33, 8)]
    short_batch = [random_prompt(vocab, 500 + n, 11 + n) for n in range(6)]
    kw = dict(page_size=64, max_seqs=12, max_model_len=4608, max_step_tokens=4608, chunk_with_decode=0,
              state_memory=24 << 20, prefix_cache=False)

    def run(**more):
        engine = engine_of(folder, dtype, **kw, **more)
        out = []
        for batch in (long_batch, short_batch):
            params = [SamplingParams(temperature=1.0, max_tokens=20, seed=500 + i) for i in range(len(batch))]
            out.append(engine.generate(batch, params))
        return engine, out

    ahead, got = run()
    assert modes_of(ahead._captured_ahead) == {"balanced", "splits"}, ahead._captured_ahead
    assert any(len(set(tokens)) > 3 for tokens in got[0])            # tokens vary: feeding a wrong one would show
    in_turn, want = run(overlap=False)
    assert not in_turn._captured_ahead and set(in_turn._graphs) == set(ahead._graphs)
    assert got == want
    if dtype == "float32":
        assert run(cuda_graphs=False)[1] == got
    ahead.built.cache.check()


def test_a_wait_that_gives_up_stops_the_engine(model):
    """Every wait inside the tcgen05 kernels is bounded and leaves a code in a word of host memory when it gives up.
    A test-only kernel makes such a wait run out (a thousand polls of a barrier at which nobody arrives: microseconds,
    and the device stays as it was); the engine reads the word after the step's completion, hands out none of the
    step's tokens, stops with the reason and refuses further work."""
    folder, config, weights, prompts = model
    engine = engine_of(folder, "bfloat16")
    kernels = engine.built.ctx.kernels
    assert kernels.status() == 0
    try:
        engine.add(prompts[0], SamplingParams(temperature=0.0, max_tokens=30))
        for _ in range(4):
            engine.step()
        kernels.status_selftest(1000)
        with pytest.raises(RuntimeError, match=r"the engine stopped: a bounded wait inside a kernel gave up .*place 15, block 0"):
            for _ in range(3):
                engine.step()
        assert kernels.status() == (15 << 28) | 1
        with pytest.raises(RuntimeError, match="the engine stopped"):
            engine.step()
        with pytest.raises(RuntimeError, match="the engine stopped"):
            engine.add([1, 2, 3])
    finally:
        assert kernels.tcgen05_status() == 0                        # (the products' and the attention's own words)
        kernels.clear_status()
    engine.close()
    healthy = engine_of(folder, "bfloat16")                         # the device and the library go on as before
    assert len(healthy.generate([prompts[0]], SamplingParams(temperature=0.0, max_tokens=4))[0]) == 4


def test_memory_is_measured_at_the_start(model):
    """Without a given size the cache pools take `memory_fraction` of what is free after the weights, less the measured
    activation peak of the largest step and of the largest step that graphs replay; the engine reports the account."""
    import torch
    folder, config, _, prompts = model
    engine = engine_of(folder, "bfloat16", state_memory=None, memory_fraction=0.02, max_step_tokens=256, max_seqs=8,
                       chunk_with_decode=32)
    memory = engine.built.memory
    assert memory.activations > 0 and memory.graphs > 0 and 0 < memory.free_before <= torch.cuda.mem_get_info()[1]
    # logits of the rows that may sample in one step are the floor of what such a step allocates
    assert memory.activations >= 8 * config["vocab_size"] * 4
    assert memory.cache <= int(memory.free_before * 0.02) - memory.activations - memory.graphs
    assert memory.cache >= 0.9 * (int(memory.free_before * 0.02) - memory.activations - memory.graphs) - (1 << 20)
    line = engine.memory_report()
    for word in ("weights", "activations", "graph pool", "cache pools", "free"):
        assert word in line
    assert "not measured" not in line
    assert len(engine.generate([prompts[1]], SamplingParams(temperature=0.0, max_tokens=4))[0]) == 4
    fixed = engine_of(folder, "bfloat16")
    assert fixed.built.memory.activations is None and "not measured" in fixed.memory_report()


@pytest.mark.parametrize("name", ["a", "b"])
@pytest.mark.parametrize("graphs", [True, False])
def test_the_engine_generates_what_the_reference_engine_generated(tmp_path, name, graphs):
    """The workloads that the reference's own engine ran on its CPU path (tests/golden/make_engine_golden.py), here on
    the GPU in true 32-bit: the same weights, prompts, pages, portions beside decoding requests and seeded temperature
    sampling give the same tokens, with the sampling kernel's hash and inverse-CDF draw."""
    from helpers import golden_engine, golden_folder
    golden = golden_engine()
    folder, config, _ = golden_folder(tmp_path, name, golden)
    work = golden["engine"][name]
    w = work["workload"]
    engine = Engine(EngineConfig(model=str(folder), dtype="float32", page_size=w["page_size"], max_seqs=w["max_seqs"],
                                 max_model_len=w["max_model_len"], max_step_tokens=w["max_step_tokens"], prefix_cache=False,
                                 chunk_with_decode=w["chunk_with_decode"], state_memory=4 << 20, cuda_graphs=graphs))
    params = [SamplingParams(temperature=w["temperature"], seed=s, max_tokens=w["max_tokens"]) for s in w["seeds"]]
    assert engine.generate(work["prompts"], params) == work["tokens"]
    engine.built.cache.check()


def test_the_sampling_kernel_draws_what_the_reference_sampler_drew():
    """`hb_sample` on the logits rows, temperatures, seeds and positions of the recorded draws."""
    import sys
    import pathlib
    import torch
    from helpers import golden_engine
    from holon_b200.kernels import load_kernels
    sys.path.insert(0, str(pathlib.Path(__file__).resolve().parent / "golden"))
    import make_engine_golden as recorded
    golden, kernels = golden_engine(), load_kernels("cuda:0")
    logits = recorded.draw_logits().to("cuda:0")
    rows = logits.shape[0]
    full = lambda v, dt: torch.full((rows,), v, dtype=dt, device="cuda:0")               # noqa: E731
    as_i32 = lambda v: torch.tensor([v], dtype=torch.int64).to(torch.int32).repeat(rows).to("cuda:0")   # noqa: E731
    for case in golden["draws"]:
        tokens = torch.zeros(rows, dtype=torch.int32, device="cuda:0")
        kernels.sample(tokens, logits, full(case["temperature"], torch.float32), full(0, torch.int32),
                       full(1.0, torch.float32), full(0.0, torch.float32), as_i32(case["seed"] & 0xFFFFFFFF),
                       as_i32(case["seed"] >> 32), full(case["position"], torch.int32), False)
        assert tokens.tolist() == case["tokens"], case
