"""The scheduler's decisions on the host, against the real cache manager on the CPU: portions under the token
budget, decode rows first in mixed steps, what happens when pages run out, and that every request finishes under
random traffic in a tight pool."""
from __future__ import annotations

import random

import pytest
import torch

from holon_b200.cache import CacheManager
from holon_b200.engine.scheduler import Request, Scheduler, Status
from holon_b200.parts import CacheEntry, PagedKV
from holon_b200.sampling import SamplingParams


def make(pages=40, max_seqs=4, max_step_tokens=16, chunk_with_decode=0, max_model_len=64):
    cache = CacheManager([CacheEntry(0, 0, PagedKV(1, 16), ())], page_size=4, max_seqs=max_seqs,
                         max_model_len=max_model_len, dtype=torch.float32, device="cpu", pages=pages)
    return Scheduler(cache, max_step_tokens, max_model_len, chunk_with_decode), cache


def request(rid, n, max_tokens=4):
    return Request(rid, list(range(n)), n, SamplingParams(temperature=0.0, max_tokens=max_tokens))


def run_step(sched, rows, finish=True):
    """What the engine does with a step's rows: advance, move prefilled requests to running, append a token, finish."""
    done = []
    for row in rows:
        r = row.request
        sched.cache.advance(r.slot, r.computed + row.n_tokens)
        sched.computed(row)
        if row.samples:
            r.tokens.append(0)
            if r.status is not Status.RUNNING:
                sched.finished_prefill(r)
            if finish and sched.at_limit(r):
                sched.finish(r, "length")
                done.append(r)
    return done


def shape(rows):
    return [(r.request.rid, r.n_tokens, r.samples) for r in rows]


def test_prefill_is_cut_under_the_budget_then_everyone_decodes():
    s, _ = make()
    for rid, n in (("a", 5), ("b", 17), ("c", 3)):
        s.add(request(rid, n))
    rows = s.schedule()
    assert shape(rows) == [("a", 5, True), ("b", 11, False)]                # 16 tokens: a whole, b's first portion
    run_step(s, rows)
    rows = s.schedule()
    assert shape(rows) == [("b", 6, True), ("c", 3, True)]                  # waiting requests go before decoding
    run_step(s, rows)
    rows = s.schedule()
    assert shape(rows) == [("a", 1, True), ("b", 1, True), ("c", 1, True)]  # oldest first
    assert [r.request.computed for r in rows] == [5, 17, 3]


def test_mixed_steps_put_decode_rows_first_and_cap_the_portion():
    s, _ = make(chunk_with_decode=6, max_step_tokens=12)
    s.add(request("a", 4))
    run_step(s, s.schedule())
    s.add(request("b", 20))
    rows = s.schedule()
    assert shape(rows) == [("a", 1, True), ("b", 6, False)] and s.mixed_steps == 1
    run_step(s, rows)
    assert shape(s.schedule()) == [("a", 1, True), ("b", 6, False)]


def test_no_slot_no_admission():
    s, _ = make(max_seqs=2)
    for rid in "abc":
        s.add(request(rid, 3))
    rows = s.schedule()
    assert shape(rows) == [("a", 3, True), ("b", 3, True)]                  # c waits for a slot
    run_step(s, rows)
    assert [r.request.rid for r in s.schedule()] == ["a", "b"]


def test_pages_run_out_lowest_ranked_is_preempted_and_recomputed():
    s, cache = make(pages=16, max_step_tokens=64)                           # 64 tokens of pool in all
    a, b = request("a", 30, max_tokens=20), request("b", 30, max_tokens=20)
    s.add(a), s.add(b)
    run_step(s, s.schedule())                                               # both prefilled: 8 pages each, pool full
    assert cache.groups[0].pool.available == 0 and [r.status for r in (a, b)] == [Status.RUNNING] * 2
    for _ in range(2):                                                      # tokens 31 and 32 fit the last pages
        run_step(s, s.schedule())
    rows = s.schedule()                                                     # a needs a ninth page: b, ranked below, goes
    assert shape(rows) == [("a", 1, True)] and s.preemptions == 1
    assert b.status is Status.PREEMPTED and b.slot == -1 and b.computed == 0 and s.waiting[0] is b
    assert len(b.tokens) == 33                                              # it keeps what it generated
    run_step(s, rows)
    cache.check()
    while a.status is not Status.FINISHED:                                  # b cannot come back while a holds the pool
        rows = s.schedule()
        assert all(r.request is a for r in rows)
        run_step(s, rows)
    rows = s.schedule()
    assert shape(rows) == [("b", 33, True)]                                 # all its tokens are computed again
    run_step(s, rows)
    assert b.status is Status.RUNNING and b.generated == 4


def test_a_running_request_with_nothing_below_it_preempts_itself():
    s, cache = make(pages=16, max_step_tokens=64, max_seqs=2)
    a, b = request("a", 31, max_tokens=30), request("b", 31, max_tokens=30)
    s.add(a), s.add(b)
    run_step(s, s.schedule())
    run_step(s, s.schedule())                                               # both at 32 tokens: the pool is full
    rows = s.schedule()                                                     # a takes b's pages; nothing is below b
    assert shape(rows) == [("a", 1, True)] and b.status is Status.PREEMPTED


@pytest.mark.parametrize("seed", range(5))
def test_random_traffic_finishes_every_request(seed):
    rng = random.Random(seed)
    s, cache = make(pages=rng.choice([16, 20, 28]), max_seqs=rng.choice([2, 3, 5]), max_step_tokens=rng.choice([8, 16, 40]),
                    chunk_with_decode=rng.choice([0, 0, 3]))
    pending = [request(f"r{i}", rng.randint(1, 40), max_tokens=rng.randint(1, 20)) for i in range(25)]
    done, steps = [], 0
    while pending or s.has_work():
        if pending and rng.random() < 0.4:
            s.add(pending.pop())
        rows = s.schedule()
        if rows is None:
            assert pending and not s.has_work()
            s.add(pending.pop())
            continue
        assert sum(r.n_tokens for r in rows) <= s.max_step_tokens
        assert len({r.request.rid for r in rows}) == len(rows)
        for r in rows:
            assert r.request.slot >= 0 and cache.capacity(r.request.slot) >= r.request.computed + r.n_tokens
        ones = [r.n_tokens == 1 and r.request.status is Status.RUNNING for r in rows]
        assert ones == sorted(ones, reverse=True)                           # decode rows come first
        done += run_step(s, rows)
        cache.check()
        steps += 1
        assert steps < 5000
    assert len(done) == 25 and all(r.generated >= 1 for r in done)
    assert not cache.live and cache.groups[0].pool.available == cache.groups[0].pool.pages


def test_a_state_that_wants_chunks_moves_the_cuts_to_their_multiples():
    """A mixer whose fixed-size state is updated in chunks of 8 tokens (`SlotState.chunk`): a portion that does not
    end its prompt ends at a multiple of 8, wherever the budget would have cut it; the portion that ends the prompt
    ends where the prompt ends; a budget too small for a whole chunk leaves the request for the next step."""
    from holon_b200.parts import SlotState
    entries = [CacheEntry(0, 0, PagedKV(1, 16), ()), CacheEntry(1, 1, None, (SlotState("sum", (4,), chunk=8),))]
    cache = CacheManager(entries, page_size=4, max_seqs=4, max_model_len=64, dtype=torch.float32, device="cpu", pages=40)
    assert cache.chunk == 8
    s = Scheduler(cache, 21, 64, 0)
    for rid, n in (("a", 30), ("b", 13), ("c", 9)):
        s.add(request(rid, n))
    rows = s.schedule()
    assert shape(rows) == [("a", 16, False)]                    # 21 tokens of budget: cut back to 16; 5 left are too few
    run_step(s, rows)                                           # for one chunk of b, whose prompt would not end there
    rows = s.schedule()
    assert shape(rows) == [("a", 14, True)]                     # the prompt's end needs no multiple; b's 7 would be none
    run_step(s, rows)
    rows = s.schedule()
    assert shape(rows) == [("b", 13, True), ("c", 8, False)]
    seen = []
    while rows:
        seen += [(r.request.rid, r.request.computed, r.n_tokens, r.samples) for r in rows]
        run_step(s, rows)
        rows = s.schedule() if s.waiting else None
    for rid, start, n, ends in seen:                            # every cut inside a prompt lies on a multiple of 8
        assert ends or (start + n) % 8 == 0, (rid, start, n)
    assert {rid for rid, _, _, ends in seen if ends} == {"b", "c"} and not s.waiting
