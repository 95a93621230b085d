"""The engine's host side on the CPU: the step function, the cache and the scheduler driven with the plain torch
kernel table of tests/ref_kernels.py in place of the CUDA kernels, against the plain implementation."""
from __future__ import annotations

import pytest
import torch

import plain_qwen3 as plain
from helpers import make_folder, random_prompt
from holon_b200.engine import Engine, EngineConfig, SamplingParams, StepEntry, StepError, build
from holon_b200.weights import SafetensorsSource
from ref_kernels import RefKernels


def built(folder, **kw):
    args = dict(dtype="float32", device="cpu", kernels=RefKernels(), page_size=4, max_seqs=4, max_model_len=128,
                max_step_tokens=64, pages=40)
    args.update(kw)
    return build(SafetensorsSource(folder), **args)


@pytest.mark.parametrize("name", ["a", "b"])
def test_whole_prompt_and_portions_match_plain(tmp_path, name):
    folder = make_folder(tmp_path, name)
    config, weights = plain.read_folder(folder)
    ids = random_prompt(config["vocab_size"], 37, 5)
    want = plain.forward(config, weights, ids)
    b = built(folder)
    slot = b.cache.admit()
    assert b.cache.reserve(slot, len(ids))
    got = b.runner.step([StepEntry(slot, ids, 0, range(len(ids)))])
    assert (got - want).abs().max() < 1e-4
    b.cache.release(slot)
    slot, at, parts = b.cache.admit(), 0, []
    for n in (5, 2, 9, 1, 1, 13, 6):
        assert b.cache.reserve(slot, at + n)
        parts.append(b.runner.step([StepEntry(slot, ids[at:at + n], at, range(n))]))
        at += n
    assert at == len(ids)
    assert (torch.cat(parts) - want).abs().max() < 1e-4
    b.cache.check()


def test_step_refuses_bad_batches(tmp_path):
    b = built(make_folder(tmp_path, "a"))
    slot = b.cache.admit()
    with pytest.raises(StepError, match="not reserved"):
        b.runner.step([StepEntry(slot, [1, 2, 3], 0)])
    b.cache.reserve(slot, 3)
    with pytest.raises(StepError, match="start at 2"):
        b.runner.step([StepEntry(slot, [1], 2)])
    with pytest.raises(StepError, match="outside the vocabulary"):
        b.runner.step([StepEntry(slot, [1, 999, 3], 0)])
    with pytest.raises(StepError, match="not admitted"):
        b.runner.step([StepEntry(3, [1], 0)])
    assert b.runner.step([StepEntry(slot, [1, 2, 3], 0)]) is None          # nothing wanted: no logits


@pytest.mark.parametrize("name,temperature", [("a", 0.0), ("b", 0.0), ("b", 0.7)])
def test_generate_matches_plain(tmp_path, name, temperature):
    folder = make_folder(tmp_path, name)
    config, weights = plain.read_folder(folder)
    prompts = [random_prompt(config["vocab_size"], n, 20 + n) for n in (5, 17, 31, 1)]
    engine = Engine(EngineConfig(model=str(folder), device="cpu", dtype="float32", page_size=4, max_seqs=3,
                                 max_model_len=64, max_step_tokens=16, chunk_with_decode=8, state_memory=1 << 20),
                    kernels=RefKernels())
    params = [SamplingParams(temperature=temperature, max_tokens=8, seed=11 + i) for i in range(len(prompts))]
    got = engine.generate(prompts, params)
    for p, g, sp in zip(prompts, got, params):
        assert g == plain.generate(config, weights, p, 8, temperature, sp.seed)
    engine.built.cache.check()
    assert not engine.built.cache.live and engine.stats()["mixed_steps"] > 0



def test_logprobs_of_generated_and_prompt_tokens(tmp_path):
    """`logprobs` and `prompt_logprobs` (core/holon/api/frontend.py:25-34): the chosen token's log-probability and the
    ranked top-k from the raw logits at every generated token; the prompt's positions 1 .. n-1 with the first delta,
    gathered over portions (and once only when the request is preempted in mid-prompt and starts again)."""
    folder = make_folder(tmp_path, "b")
    config, weights = plain.read_folder(folder)
    prompts = [random_prompt(config["vocab_size"], n, 40 + n) for n in (23, 9, 1)]
    engine = Engine(EngineConfig(model=str(folder), device="cpu", dtype="float32", page_size=4, max_seqs=3,
                                 max_model_len=64, max_step_tokens=16, chunk_with_decode=8, state_memory=1 << 20),
                    kernels=RefKernels())
    params = [SamplingParams(temperature=0.8, max_tokens=5, seed=3, logprobs=3, prompt_logprobs=2),
              SamplingParams(temperature=0.0, max_tokens=5, logprobs=0),
              SamplingParams(temperature=0.0, max_tokens=5, prompt_logprobs=0, n=2)]
    rids = [engine.add(p, sp) for p, sp in zip(prompts, params)]
    seen: dict = {}
    while engine.has_work():
        for d in engine.step():
            seen.setdefault((d.rid, d.index), []).append(d)
    for rid, prompt, sp in zip(rids, prompts, params):
        for index in range(sp.n):
            deltas = seen[(rid, index)]
            ids = list(prompt)
            first = deltas[0].prompt_logprobs
            assert all(d.prompt_logprobs is None for d in deltas[1:])
            if sp.prompt_logprobs is None or index:
                assert first is None
            else:
                whole = plain.forward(config, weights, ids)
                assert len(first.token) == len(first.top) == len(first.top_ids) == len(ids) - 1
                for at in range(len(ids) - 1):
                    own, top_ids, top = plain.logprobs(whole[at], ids[at + 1], sp.prompt_logprobs)
                    assert abs(first.token[at] - own) < 1e-4 and first.top_ids[at] == top_ids
                    assert all(abs(a - b) < 1e-4 for a, b in zip(first.top[at], top))
            for d in deltas:
                logits = plain.forward(config, weights, ids)[-1]
                if sp.logprobs is None:
                    assert d.logprobs is None
                else:
                    own, top_ids, top = plain.logprobs(logits, d.token_ids[0], sp.logprobs)
                    assert abs(d.logprobs.token[0] - own) < 1e-4 and d.logprobs.top_ids == [top_ids]
                    assert all(abs(a - b) < 1e-4 for a, b in zip(d.logprobs.top[0], top))
                ids += d.token_ids
    with pytest.raises(ValueError, match="logprobs"):
        engine.add([1], SamplingParams(logprobs=-1))
    engine.built.cache.check()
    assert not engine.built.cache.live and not engine._prompt_lp


def test_which_steps_are_kept_as_graphs(tmp_path):
    """The shapes `Engine._graph_fits` accepts: one-token rows alone up to the largest bucket, or beside one or two
    prompt portions that fill `chunk_with_decode` exactly."""
    folder = make_folder(tmp_path, "a")
    engine = Engine(EngineConfig(model=str(folder), device="cpu", dtype="float32", page_size=4, max_seqs=3,
                                 max_model_len=64, max_step_tokens=16, chunk_with_decode=8, state_memory=1 << 20),
                    kernels=RefKernels())
    one = lambda slot: StepEntry(slot, [1], 0)                       # noqa: E731
    part = lambda slot, n: StepEntry(slot, list(range(n)), 0)        # noqa: E731
    fits = lambda entries: engine._graph_fits(entries, sum(len(e.tokens) == 1 for e in entries))   # noqa: E731
    assert engine._buckets == (1, 2, 3)                              # max_seqs itself is the last bucket
    assert fits([one(0)]) and fits([one(0), one(1), one(2)])
    assert not fits([one(0), one(1), one(2), one(3)])               # more rows than the largest bucket
    assert fits([one(0), part(1, 8)]) and fits([one(0), part(1, 5), part(2, 3)])
    assert not fits([one(0), part(1, 7)])                           # the budget is not filled
    assert not fits([part(1, 8)])                                   # no decode row beside it: a plain prefill step
    assert not fits([one(0), part(1, 2), part(2, 3), part(3, 3)])   # three portions
    engine.config.chunk_with_decode = 0
    assert not fits([one(0), part(1, 8)]) and fits([one(0)])


def test_prefix_cache_gives_the_same_tokens_and_skips_the_shared_pages(tmp_path):
    """Prompts with equal beginnings through an engine with the prefix cache and one without: the same tokens (32-bit),
    fewer prompt tokens computed, `cached_tokens` on every request's first delta; the sequences of an `n` = 3
    request start on the first one's pages; a pool too small for all requests (preemption, eviction) changes nothing."""
    folder = make_folder(tmp_path, "b")
    config, weights = plain.read_folder(folder)
    stem = random_prompt(config["vocab_size"], 22, 3)
    prompts = [stem + random_prompt(config["vocab_size"], n, 50 + n) for n in (1, 6, 13)] + [stem[:9], stem]
    params = SamplingParams(temperature=0.7, max_tokens=6, seed=5)

    def run(prompts=prompts, params=params, **kw):
        args = dict(model=str(folder), device="cpu", dtype="float32", page_size=4, max_seqs=3, max_model_len=64,
                    max_step_tokens=16, chunk_with_decode=8, state_memory=1 << 20)
        args.update(kw)
        engine = Engine(EngineConfig(**args), kernels=RefKernels())
        out, cached = {}, {}
        for round_ in range(2):                                      # the second round finds the first one's pages kept
            rids = [engine.add(p, params) for p in prompts]
            while engine.has_work():
                for d in engine.step():
                    out.setdefault((round_, d.rid), []).extend(d.token_ids)
                    if d.cached_tokens is not None:
                        assert (round_, d.rid) not in cached
                        cached[(round_, d.rid)] = d.cached_tokens
            engine.built.cache.check()
            assert not engine.built.cache.live
        return engine, [out[k] for k in sorted(out)], cached

    plain_engine, want, cached = run(prefix_cache=False)
    assert plain_engine.built.cache.prefix is None and set(cached.values()) == {0}
    for p, got in zip(prompts, want[:len(prompts)]):
        assert got == plain.generate(config, weights, p, 6, 0.7, 5)
    engine, got, cached = run()
    assert got == want
    stats = engine.stats()
    assert stats["prefix_hit_tokens"] > 0 and len(cached) == 2 * len(prompts)
    assert all(c % 4 == 0 for c in cached.values()) and max(cached.values()) >= 20
    second_round = [c for (r, _), c in cached.items() if r == 1]
    assert all(c >= 8 for c in second_round)                         # everyone finds at least the stem's beginning
    long = SamplingParams(temperature=0.7, max_tokens=30, seed=5)     # 16 pages of 4,608 bytes: one request of 64 tokens
    small, got_small, _ = run(prompts[:3], long, state_memory=17 * 4608)
    assert small.built.cache.pages == 16 and small.stats()["preemptions"] > 0 and small.stats()["prefix_hit_tokens"] > 0
    assert got_small == run(prompts[:3], long, prefix_cache=False)[1]

    engine = Engine(EngineConfig(model=str(folder), device="cpu", dtype="float32", page_size=4, max_seqs=3,
                                 max_model_len=64, max_step_tokens=16, chunk_with_decode=8, state_memory=1 << 20),
                    kernels=RefKernels())
    rid = engine.add(stem, SamplingParams(temperature=0.7, max_tokens=4, seed=9, n=3))
    first: dict[int, int] = {}
    while engine.has_work():
        for d in engine.step():
            if d.cached_tokens is not None:
                first[d.index] = d.cached_tokens
    assert first == {0: 0, 1: 20, 2: 20} and rid not in engine.requests
    engine.add(stem, SamplingParams(max_tokens=4, n=2), rid="gone")
    engine.step()
    assert sorted(d.index for d in engine.abort("gone")) == [0, 1]   # the second sequence had not started
    engine.drain()
    assert not engine.has_work() and not engine.built.cache.live and not engine._siblings


@pytest.mark.parametrize("seed", range(3))
def test_random_arrivals_aborts_and_a_small_pool(tmp_path, seed):
    """Requests from a few prompt families arrive at random steps, some are aborted in mid-flight, the pool holds one
    request of the longest length and a little more: whatever is preempted, evicted or shared, every request that
    finishes has the plain implementation's tokens, and in the end nothing is held."""
    import random
    rng = random.Random(seed)
    folder = make_folder(tmp_path, "a")
    config, weights = plain.read_folder(folder)
    page_bytes = 2 * 2 * 2 * 4 * 16 * 4                              # layers x (k, v) x kv heads x page x head size x 4 bytes
    engine = Engine(EngineConfig(model=str(folder), device="cpu", dtype="float32", page_size=4, max_seqs=4,
                                 max_model_len=48, max_step_tokens=24, chunk_with_decode=rng.choice([0, 8]),
                                 state_memory=(12 + rng.choice([1, 4, 9])) * page_bytes + page_bytes),
                    kernels=RefKernels())
    families = [random_prompt(config["vocab_size"], 30, 70 + i) for i in range(3)]
    pending = []
    for i in range(14):
        prompt = families[rng.randrange(3)][:rng.choice([3, 8, 13, 21, 30])] + random_prompt(config["vocab_size"], rng.randrange(4), 200 + i)
        pending.append((rng.randrange(25), f"q{i}", prompt, SamplingParams(temperature=0.6, seed=i, max_tokens=rng.choice([1, 5, 12]))))
    got: dict[str, list[int]] = {}
    done, aborted, asked, step = set(), set(), {}, 0
    while pending or engine.has_work():
        for item in [p for p in pending if p[0] <= step]:
            pending.remove(item)
            asked[engine.add(item[2], item[3], rid=item[1])] = item
        if asked and rng.random() < 0.08:
            victim = rng.choice(sorted(asked))
            if victim not in done and victim not in aborted and engine.abort(victim):
                aborted.add(victim)
        for d in engine.step():
            assert d.rid not in aborted
            got.setdefault(d.rid, []).extend(d.token_ids)
            if d.finish_reason:
                done.add(d.rid)
        engine.built.cache.check()
        step += 1
        assert step < 2000
    assert done | aborted == set(asked) and not done & aborted
    for rid in done:
        _, _, prompt, sp = asked[rid]
        assert got[rid] == plain.generate(config, weights, prompt, sp.max_tokens, 0.6, sp.seed), rid
    assert not engine.built.cache.live and engine.built.cache.free_tokens() == engine.built.cache.pages * 4
    stats = engine.stats()
    assert stats["preemptions"] > 0 and stats["prefix_hit_tokens"] > 0      # (seeds chosen so that both happen)


def test_layout_of_a_step_that_runs_as_a_graph(tmp_path):
    """`Runner.context(entries, pad_rows=...)`: one-token rows first in their order, then the padding rows (padding
    slot, position 0, kv_len 1), then the prompt portions; logits at the last token of every row."""
    b = built(make_folder(tmp_path, "a"), max_seqs=6)
    slots = [b.cache.admit() for _ in range(4)]
    for slot, n in zip(slots, (9, 1, 30, 12)):
        assert b.cache.reserve(slot, n)
    b.cache.advance(slots[0], 8)                                     # slot 0 holds 8 tokens and decodes
    b.cache.advance(slots[2], 20)                                    # slot 2 is in mid-prompt
    entries = [StepEntry(slots[2], list(range(5)), 20, ()), StepEntry(slots[0], [7], 8, (0,)),
               StepEntry(slots[3], list(range(3)), 0, (2,)), StepEntry(slots[1], [9], 0, (0,))]
    step = b.runner.context(entries, pad_rows=2, extra={"sample_slot": torch.arange(6, dtype=torch.int32).numpy()})
    rows = step.rows
    assert (rows.n_rows, rows.n_tokens, rows.n_decode, rows.max_q) == (6, 12, 4, 5)
    assert rows.row_slot.tolist() == [slots[0], slots[1], b.cache.padding_slot, b.cache.padding_slot, slots[2], slots[3]]
    assert rows.query_start.tolist() == [0, 1, 2, 3, 4, 9, 12] and rows.kv_len.tolist() == [9, 1, 1, 1, 25, 3]
    assert step.token_ids.tolist() == [7, 9, 0, 0, 0, 1, 2, 3, 4, 0, 1, 2]
    assert step.positions.tolist() == [8, 0, 0, 0, 20, 21, 22, 23, 24, 0, 1, 2]
    assert step.logits_index.tolist() == [0, 1, 2, 3, 8, 11]
    assert step.offset_of == {1: 0, 3: 1, 0: 4, 2: 9}
    null = b.cache.groups[0].null_page * 4
    write = step.groups[0].write_index.tolist()
    assert write[2] // 4 * 4 == null and write[3] // 4 * 4 == null   # the padding rows write into the null page
    assert write[0] == int(b.cache.groups[0].table[slots[0], 2]) * 4 + 0


def test_the_engine_stops_when_a_kernel_reports_a_wait_that_gave_up(tmp_path):
    """The kernel table's `status()` is read after every step's completion and before its tokens are handed out: a
    non-zero word stops the engine with the reason, and it takes no further work
    (core/holon/core/engine.py:498-499, 607-612)."""
    class Flaky(RefKernels):
        word = 0

        def status(self):
            return self.word

    kernels = Flaky()
    engine = Engine(EngineConfig(model=str(make_folder(tmp_path, "a")), device="cpu", dtype="float32", page_size=4,
                                 max_seqs=3, max_model_len=64, max_step_tokens=16, state_memory=1 << 20),
                    kernels=kernels)
    engine.add([1, 2, 3], SamplingParams(temperature=0.0, max_tokens=8))
    engine.step()                                                    # (depth 1: its tokens come a step later)
    assert [d.token_ids for d in engine.step()]
    kernels.word = (2 << 28) | 6
    with pytest.raises(RuntimeError, match=r"stopped: a bounded wait.*place 2, block 5"):
        for _ in range(3):
            engine.step()
    with pytest.raises(RuntimeError, match="the engine stopped"):
        engine.step()
    with pytest.raises(RuntimeError, match="the engine stopped"):
        engine.add([4, 5])
    engine.close()                                                   # still closes


def test_block_table_rows_travel_as_copies_with_the_step(tmp_path):
    """Rows of the block table that changed go to the device inside the step's own upload, as copies taken when the
    step is laid out: what the host does to its table afterwards (a window letting go of pages, a request ending)
    cannot reach a step that is already on its way."""
    b = built(make_folder(tmp_path, "a"))
    group = b.cache.groups[0]
    slot = b.cache.admit()
    assert b.cache.reserve(slot, 10)
    slots, rows = group.take_dirty()
    assert slots.tolist() == [slot] and rows[0, :3].tolist() == group.table[slot, :3].tolist()
    before = rows.copy()
    b.cache.release(slot)                                            # the host table moves on
    assert (rows == before).all() and (group.table[slot] == group.null_page).all()
    assert group.take_dirty()[0].tolist() == [slot] and group.take_dirty()[0].tolist() == []
    slot = b.cache.admit()
    assert b.cache.reserve(slot, 6)
    b.runner.step([StepEntry(slot, [1, 2, 3, 4, 5, 6], 0)])
    assert group.table_device[slot].tolist() == group.table[slot].tolist()
    assert b.runner.uploader.bytes_last >= 4 * (1 + group.max_pages)  # counted with the step's upload


@pytest.mark.parametrize("name", ["a", "b"])
def test_the_engine_generates_what_the_reference_engine_generated(tmp_path, name):
    """The workloads that the reference's own engine ran on the CPU (tests/golden/make_engine_golden.py): the same
    weights, prompts, pages, portions beside decoding requests and seeded temperature sampling give the same tokens,
    also in a pool so small that requests are preempted and computed again."""
    from helpers import golden_engine, golden_folder
    golden = golden_engine()
    folder, config, _ = golden_folder(tmp_path, name, golden)
    work = golden["engine"][name]
    w = work["workload"]
    page_bytes = config["num_hidden_layers"] * 2 * config["num_key_value_heads"] * w["page_size"] * config["head_dim"] * 4
    for pages, overlap in ((64, False), (-(-w["max_model_len"] // w["page_size"]) + 2, True)):
        engine = Engine(EngineConfig(model=str(folder), device="cpu", dtype="float32", page_size=w["page_size"],
                                     max_seqs=w["max_seqs"], max_model_len=w["max_model_len"], prefix_cache=False,
                                     max_step_tokens=w["max_step_tokens"], chunk_with_decode=w["chunk_with_decode"],
                                     state_memory=page_bytes * (pages + 1), overlap=overlap), kernels=RefKernels())
        params = [SamplingParams(temperature=w["temperature"], seed=s, max_tokens=w["max_tokens"]) for s in w["seeds"]]
        assert engine.generate(work["prompts"], params) == work["tokens"]
        assert engine.stats()["mixed_steps"] > 0
        engine.built.cache.check()


def test_prefix_cache_with_windowed_layers_beside_full_ones():
    """A toy model with two cache groups (layers that see all keys, layers that see the last 10): with the prefix cache
    requests start in the middle of their prompts in both groups, holding in the windowed group only the pages that
    reach into the window, and generate what an engine without the prefix cache generates; also in a pool so small
    that requests are preempted and kept pages evicted."""
    from holon_b200.config import register_architecture, unregister_architecture
    from holon_b200.weights import RandomSource
    from test_gpu_toy_parts import window_recipe
    register_architecture("ToyWindowPrefixForCausalLM", dict, window_recipe)
    try:
        config = {"architectures": ["ToyWindowPrefixForCausalLM"], "hidden": 32, "vocab": 61, "inter": 48, "head_dim": 16,
                  "window": 10}
        stem = random_prompt(61, 30, 3)
        prompts = [stem + random_prompt(61, n, 50 + n) for n in (1, 6, 13)] + [stem[:13], stem]

        def run(max_tokens=6, **kw):
            args = dict(model="toy", device="cpu", dtype="float32", page_size=4, max_seqs=3, max_model_len=80,
                        max_step_tokens=16, chunk_with_decode=8, state_memory=1 << 20)
            args.update(kw)
            engine = Engine(EngineConfig(**args), source=RandomSource(config, seed=8, dtype=torch.float32),
                            kernels=RefKernels())
            params = SamplingParams(temperature=0.8, max_tokens=max_tokens, seed=11)
            out, cached = {}, {}
            for round_ in range(2):
                rids = [engine.add(p, params) for p in prompts]
                while engine.has_work():
                    for d in engine.step():
                        out.setdefault((round_, d.rid), []).extend(d.token_ids)
                        if d.cached_tokens is not None:
                            cached[(round_, d.rid)] = d.cached_tokens
                    engine.built.cache.check()
                assert not engine.built.cache.live and len(rids) == len(prompts)
            return engine, [out[k] for k in sorted(out)], cached

        plain_engine, want, _ = run(prefix_cache=False)
        assert len(plain_engine.built.cache.groups) == 2 and plain_engine.built.cache.prefix is None
        engine, got, cached = run()
        assert engine.built.cache.prefix is not None and engine.built.cache.prefix.windows == (10, 0)
        assert got == want and any(len(set(t)) > 2 for t in got)
        assert engine.stats()["prefix_hit_tokens"] > 0 and max(cached.values()) >= 28
        assert all(c >= 12 for (r, _), c in cached.items() if r == 1)
        per_page = sum(g.kv[:, 0].numel() * 4 for g in engine.built.cache.groups)
        small, got_small, _ = run(max_tokens=30, state_memory=21 * per_page)
        assert small.built.cache.pages == 20 and small.stats()["preemptions"] > 0 and small.stats()["prefix_hit_tokens"] > 0
        assert got_small == run(max_tokens=30, prefix_cache=False)[1]
    finally:
        unregister_architecture("ToyWindowPrefixForCausalLM")
