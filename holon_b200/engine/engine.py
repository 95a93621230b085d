"""The engine a user calls: requests in, tokens out.

`Engine(EngineConfig(model=...)).generate(prompts, params)` returns the generated token ids of each prompt;
`add` / `step` / `has_work` / `abort` / `stats` / `close` drive it by hand. Names and meanings follow the reference
(core/holon/core/engine.py:332-376, 461-524, 702-709). With `overlap` (the default) a step stays in flight while
the host schedules and enqueues the next one; without it every step is read back before the next is scheduled.
"""
from __future__ import annotations

import dataclasses
import secrets
from collections.abc import Sequence

import numpy as np
import torch

from ..config.engine import EngineConfig
from ..sampling import Sampler, SamplingParams, sampling_arrays, sequence_seed
from ..weights import SafetensorsSource
from .batch import StepEntry
from .build import build
from .scheduler import Request, Row, Scheduler, Status

GRAPH_BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)
GRAPH_PORTIONS = 2                            # prompt portions beside the decode rows of a step that runs as a graph


@dataclasses.dataclass
class Logprobs:
    """Per position: the chosen token's log-probability and the ranked top-k (ids and log-probabilities as parallel
    lists), from the raw logits, before temperature and filters. Prompt logprobs cover prompt positions 1 .. n-1: the
    first token has no context (core/holon/api/frontend.py:25-34)."""

    token: list[float]
    top_ids: list[list[int]]
    top: list[list[float]]


@dataclasses.dataclass
class TokenDelta:
    """What one step added to one request (core/holon/api/frontend.py:41-52)."""

    rid: str
    token_ids: list[int]
    index: int = 0                           # which of the request's `n` sequences these belong to
    logprobs: Logprobs | None = None         # of these tokens, where the request asked for them
    prompt_logprobs: Logprobs | None = None  # of the prompt, with the sequence's first delta
    finish_reason: str | None = None         # "stop" | "length" | "abort" | None
    cached_tokens: int | None = None         # on a sequence's first delta: prompt tokens the prefix cache served


PROMPT_LOGPROB_ROWS = 256                     # rows of full-vocabulary logits held at once for prompt logprobs


@dataclasses.dataclass
class _Inflight:
    """A launched step: its rows, the ones that sample, where their tokens will land on the host, and the event that
    says they have."""

    rows: list
    sampled: list
    host: torch.Tensor | None
    done: object
    decode_only: bool
    pick: list | None = None                 # where in `host` each sampled row's token lies (None: in their order)
    logprobs: tuple | None = None            # host tensors (chosen, top ids, top) for the sampled rows, in their order
    prompt: list = dataclasses.field(default_factory=list)   # (request, k, host chosen, host top ids, host top) pieces


class Engine:
    def __init__(self, config: EngineConfig, source=None, kernels=None) -> None:
        """`source`: a weight source in place of the folder `config.model` (random weights, for one);
        `kernels`: a kernel table in place of the compiled CUDA kernels (tests on a machine without a GPU)."""
        self.config = config
        source = source or SafetensorsSource(config.model)
        self.built = build(source, dtype=config.dtype, device=config.device, kernels=kernels,
                           page_size=config.page_size, max_seqs=config.max_seqs, max_model_len=config.max_model_len,
                           max_step_tokens=config.max_step_tokens, state_memory=config.state_memory,
                           memory_fraction=config.memory_fraction, prefix_cache=config.prefix_cache,
                           chunk_with_decode=config.chunk_with_decode, cuda_graphs=config.cuda_graphs)
        b = self.built
        self.device = b.ctx.device
        self.eos = frozenset(source.eos_token_ids())
        self.scheduler = Scheduler(b.cache, config.max_step_tokens, config.max_model_len, config.chunk_with_decode)
        self.sampler = Sampler(b.ctx.kernels, self.device)
        self.requests: dict[str, list[Request]] = {}          # a request's sequences that have not finished
        self._prompt_lp: dict[Request, Logprobs] = {}         # sequences whose prompt logprobs are still being gathered
        self._siblings: dict[Request, list[Request]] = {}     # sequences that wait for their request's first one's prompt
        self._base_seed = config.seed if config.seed is not None else secrets.randbits(63)
        self._added = 0
        self._graphs: dict[tuple, tuple] = {}
        self._captured_ahead: set[tuple] = set()               # keys of graphs captured with rows fed from the device
        self._graph_pool = None
        self._use_graphs = config.cuda_graphs and self.device.type == "cuda"
        self._buckets = tuple(x for x in GRAPH_BUCKETS if x < config.max_seqs) + (config.max_seqs,)   # the fullest batch too
        self._host_tokens = [torch.zeros(config.max_seqs + 1 + GRAPH_PORTIONS, dtype=torch.int32) for _ in range(2)]
        if self.device.type == "cuda":
            self._host_tokens = [t.pin_memory() for t in self._host_tokens]
        self._flip = 0
        self._inflight: _Inflight | None = None
        self._stopped: str | None = None                       # why the engine stopped: a kernel's bounded wait gave up
        # the token each request sampled last, by slot, on the device: decode rows of a step that is enqueued before
        # the step ahead of it has been read back take their input from here
        self.last_tokens = torch.zeros(config.max_seqs + 1, dtype=torch.int32, device=self.device)
        self.steps = self.graph_steps = self.mixed_graph_steps = self._graph_launches = 0
        self.h2d_bytes = self.d2h_bytes = 0

    # ------------------------------------------------------------------ requests
    def add(self, token_ids: Sequence[int], params: SamplingParams | None = None, rid: str | None = None) -> str:
        """Queues a request. Its `params.n` sequences stream as TokenDeltas with `index` 0 .. n-1, each sampling from
        a seed of its own (core/holon/core/engine.py:331-376). With the prefix cache the sequences after the first
        wait until the first one's prompt is cached and start on its pages; without it each computes the prompt."""
        if self._stopped:
            raise RuntimeError(f"the engine stopped: {self._stopped}")
        params = params or SamplingParams()
        params.validate()
        tokens = [int(t) for t in token_ids]
        if not tokens:
            raise ValueError("empty prompt")
        if len(tokens) >= self.config.max_model_len:
            raise ValueError(f"prompt of {len(tokens)} tokens leaves no room under max_model_len "
                             f"{self.config.max_model_len}")
        vocab = self.built.model.spec.vocab
        if any(not 0 <= t < vocab for t in tokens):
            raise ValueError(f"a prompt token is outside the vocabulary of {vocab}")
        rid = rid if rid is not None else f"r{self._added}"
        if rid in self.requests:
            raise ValueError(f"request id {rid!r} is in use")
        base = params.seed if params.seed is not None else sequence_seed(self._base_seed, self._added + 1)
        self._added += 1
        self.requests[rid] = live = []
        for i in range(params.n):
            live.append(Request(rid, list(tokens), len(tokens), params, sequence_seed(base, i), index=i))
            if i == 0 and params.prompt_logprobs is not None:      # once a request (core/holon/core/engine.py:360-366)
                self._prompt_lp[live[-1]] = Logprobs([], [], [])
            if i == 0 or self.built.cache.prefix is None:
                self.scheduler.add(live[-1])
            else:                  # siblings wait until the first sequence's prompt is cached, then start on its pages
                self._siblings.setdefault(live[0], []).append(live[-1])
        return rid

    def abort(self, rid: str) -> list[TokenDelta]:
        """Finishes every sequence of request `rid` that is still live, one delta each; none if the id is unknown
        (core/holon/core/engine.py:391-410)."""
        deltas = []
        live = self.requests.pop(rid, [])
        held = {id(sibling) for first in live for sibling in self._siblings.pop(first, [])}   # never started: nothing to release
        for request in live:
            if id(request) in held:
                request.status, request.finish_reason = Status.FINISHED, "abort"
            else:
                self.scheduler.finish(request, "abort", release=request.pending == 0)   # (a row in flight gives the slot back)
            self._prompt_lp.pop(request, None)
            deltas.append(TokenDelta(rid, [], request.index, finish_reason="abort"))
        return deltas

    def has_work(self) -> bool:
        return self.scheduler.has_work() or self._inflight is not None

    # ------------------------------------------------------------------ one step
    def step(self) -> list[TokenDelta]:
        """Runs one step and returns what became known. With `overlap`, the step launched here stays in flight and
        the deltas are those of the step before it: the host schedules and enqueues step N + 1 while step N runs,
        decode rows reading their input token from the device (core/holon/core/engine.py:492-524)."""
        if self._stopped:
            raise RuntimeError(f"the engine stopped: {self._stopped}")
        deltas: list[TokenDelta] = []
        prev, self._inflight = self._inflight, None
        if prev is not None and not self._may_run_ahead(prev):
            deltas += self._commit(prev)
            prev = None
        rows = self.scheduler.schedule()
        if rows is None and prev is not None:
            deltas += self._commit(prev)
            prev = None
            rows = self.scheduler.schedule()
        if rows is None:
            if self.scheduler.has_work():
                raise RuntimeError("the scheduler made no progress with requests pending")
            return deltas
        current = self._launch(rows)
        if prev is not None:
            deltas += self._commit(prev)
        if self.config.overlap:
            self._inflight = current
        else:
            deltas += self._commit(current)
        return deltas

    def drain(self) -> list[TokenDelta]:
        """Commits the step in flight, if any."""
        prev, self._inflight = self._inflight, None
        return self._commit(prev) if prev is not None else []

    def _may_run_ahead(self, prev: "_Inflight") -> bool:
        """Whether the next step can be scheduled before `prev` is committed: `prev` was a pure decode step over every
        running request, nobody waits, nobody is at its limit, and every request's next token has a page without
        taking one from another request. Then the next step is the same rows again, fed from the device, and no
        scheduling decision depends on the tokens still in flight (a stop token costs one wasted row)."""
        s = self.scheduler
        if not prev.decode_only or s.waiting or len(prev.rows) != len(s.running):
            return False
        need = 0
        for row in prev.rows:
            r = row.request
            if r.status is not Status.RUNNING or s.at_limit(r):
                return False
            need += r.computed + 1 > self.built.cache.capacity(r.slot)
        return need == 0 or all(g.pool.available >= need for g in self.built.cache.groups)

    def _launch(self, rows: list[Row]) -> "_Inflight":
        """Enqueues a step: forward, sampling, the sampled tokens filed by slot on the device and copied to the host."""
        runner = self.built.runner
        entries = []
        for r in rows:
            q = r.request
            if q.pending:                                  # its last token is still on the device
                entries.append(StepEntry(q.slot, (0,), q.computed, (0,) if r.samples else (), from_last=True))
            else:
                entries.append(StepEntry(q.slot, q.tokens[q.computed:q.computed + r.n_tokens], q.computed,
                                         (r.n_tokens - 1,) if r.samples else ()))
        sampled = [r for r in rows if r.samples]
        n = len(sampled)
        runner.check(entries)
        ones = sum(1 for e in entries if len(e.tokens) == 1)
        decode_only = n == ones == len(entries)
        host = pick = lps = None
        owed = self._prompt_rows(rows) if self._prompt_lp else []
        if n:
            arrays = sampling_arrays([(r.request.params, r.request.seed, r.request.computed + r.n_tokens)
                                      for r in sampled])
            arrays["sample_slot"] = np.array([r.request.slot for r in sampled], dtype=np.int32)
            filtered = any(r.request.params.filtered for r in sampled)
            ks = [r.request.params.logprobs for r in sampled if r.request.params.logprobs is not None]
            if self._use_graphs and not filtered and not ks and not owed and self._graph_fits(entries, ones):
                tokens, pick = self._replay(entries, [r.samples for r in rows], arrays)      # (graphs return tokens only)
                m = tokens.shape[0]
                if pick == list(range(n)):                 # (a plain decode step: its n tokens lie first, in order)
                    m, pick = n, None
            else:
                step = runner.context(entries, extra=arrays)
                tokens, lps, owed = self._forward(step, filtered, n, logprobs=max(ks) if ks else None, prompt=owed)
                m = n
            host = self._host_tokens[self._flip][:m]
            self._flip ^= 1
            host.copy_(tokens[:m], non_blocking=True)
            self.d2h_bytes += m * 4
        else:                                              # every row stops short of its prompt's end: the head is skipped
            step = runner.context(entries)
            _, _, owed = self._forward(step, False, 0, prompt=owed)
        self.h2d_bytes += runner.uploader.bytes_last
        done = None
        if self.device.type == "cuda":
            done = torch.cuda.Event()
            done.record()
        runner.commit(entries)                             # the cache's books: these tokens are (being) computed
        for r in rows:
            self.built.cache.publish(r.request.slot, r.request.tokens)   # whole pages of known tokens: shareable from now on
            self.scheduler.computed(r)
            r.request.pending += int(r.samples)
        self.steps += 1
        return _Inflight(rows, sampled, host, done, decode_only, pick, lps, owed)

    def _prompt_rows(self, rows: list[Row]) -> list[tuple]:
        """The prompt logprobs this step's rows owe: (entry, request, first and end offset among its tokens, targets)
        for the prompt positions they compute that predict a prompt token, except those already recorded (a request
        preempted in mid-prompt computes them again) (core/holon/core/engine.py:588-602)."""
        out = []
        for i, r in enumerate(rows):
            q = r.request
            acc = self._prompt_lp.get(q)
            if acc is None or q.pending:
                continue
            lo, hi = max(q.computed, len(acc.token)), min(q.computed + r.n_tokens, q.prompt_len - 1)
            if lo < hi:
                out.append((i, q, lo - q.computed, hi - q.computed, q.tokens[lo + 1:hi + 1]))
        return out

    def _graph_fits(self, entries, ones: int) -> bool:
        """Whether the step's shape is one that graphs are kept for: rows of one token alone, up to the largest
        bucket; or such rows beside one or two prompt portions that fill the budget `chunk_with_decode` exactly, which
        is what a step looks like while prompts wait behind decoding requests. (A graph serves every step with the
        same counts; other shapes come too rarely to be worth a capture.)"""
        if ones > self._buckets[-1]:
            return False
        portions = len(entries) - ones
        if portions == 0:
            return True
        c = self.config.chunk_with_decode
        return 0 < c and ones > 0 and portions <= GRAPH_PORTIONS \
            and sum(len(e.tokens) for e in entries) - ones == c

    def _feed(self, step) -> None:
        self.built.ctx.kernels.feed_tokens(step.token_ids, self.last_tokens, step.rows, step.from_last)

    def _forward(self, step, filtered: bool, n: int, out: torch.Tensor | None = None, logprobs: int | None = None,
                 prompt: list | None = None):
        """feed -> model -> sample -> store, all enqueued. Returns the device tensor of the `n` sampled tokens (None
        when nothing is sampled: the head is skipped), the sampled rows' logprobs on their way to the host (`logprobs`
        not None: that many top entries), and the pieces of `prompt`'s logprobs on their way to the host."""
        self._feed(step)
        model = self.built.runner.model
        stream = model.trunk(step)
        tokens = lps = None
        if n:
            logits = model.logits_at(stream, step.logits_index)
            tokens = self.sampler.sample(logits, step.extra, filtered, out)
            self.built.ctx.kernels.store_tokens(self.last_tokens, step.extra["sample_slot"], tokens, n)
            if logprobs is not None:
                lps = self._to_host(self.sampler.logprobs(logits, tokens, logprobs))
        pieces = []
        for i, q, a, b, targets in prompt or []:           # a bounded number of full-vocabulary rows at a time
            k, at = q.params.prompt_logprobs, step.offset_of[i]
            for c in range(a, b, PROMPT_LOGPROB_ROWS):
                d = min(b, c + PROMPT_LOGPROB_ROWS)
                index = torch.arange(at + c, at + d, dtype=torch.int32, device=self.device)
                want = torch.tensor(targets[c - a:d - a], dtype=torch.int32).to(self.device, non_blocking=True)
                got = self.sampler.logprobs(model.logits_at(stream, index), want, k)
                pieces.append((q, *self._to_host(got)))
        return tokens, lps, pieces

    def _to_host(self, tensors) -> tuple:
        out = []
        for t in tensors:
            host = torch.empty(t.shape, dtype=t.dtype, pin_memory=self.device.type == "cuda")
            host.copy_(t, non_blocking=True)
            self.d2h_bytes += t.numel() * t.element_size()
            out.append(host)
        return tuple(out)

    def _replay(self, entries, samples, arrays) -> tuple[torch.Tensor, list[int]]:
        """A step through the CUDA graph of its shape (core/holon/core/executor.py:316-344). One-token rows are padded
        to a bucket with rows of the padding slot, which read and write the null page; prompt portions follow. Every
        row's last token is sampled (a row that does not want it files the token under the padding slot), so that
        the work depends on the shape alone. Returns the tokens of all rows and, for each sampling entry in the
        entries' order, its row."""
        runner, cache = self.built.runner, self.built.cache
        single = [i for i, e in enumerate(entries) if len(e.tokens) == 1]
        portions = [i for i, e in enumerate(entries) if len(e.tokens) != 1]
        bucket = next(b for b in self._buckets if b >= len(single))
        pad, m = bucket - len(single), bucket + len(portions)
        row_of = {i: r for r, i in enumerate(single)} | {i: bucket + r for r, i in enumerate(portions)}
        wanted = [i for i, s in enumerate(samples) if s]
        at = np.array([row_of[i] for i in wanted], dtype=np.int64)
        padded = {}
        for name, values in arrays.items():
            full = np.full(m, cache.padding_slot if name == "sample_slot" else 0, dtype=values.dtype)
            full[at] = values
            padded[name] = full
        step = runner.context(entries, pad_rows=pad, extra=padded)
        kernels = self.built.ctx.kernels
        # what the mixers' kernels pin for a captured step is part of the key: a graph per plan
        key = (bucket, len(portions), step.rows.n_tokens - bucket, runner.model.capture_plan(step, self.config.max_model_len))
        if key not in self._graphs:
            # The first step of a shape runs eagerly (which also warms up what the capture must not do for the first
            # time) and is then recorded for the steps to come. Its results are the eager run's: replaying the new
            # graph on top would run the step twice, and the second run would feed on what the first one stored.
            out = torch.empty(m, dtype=torch.int32, device=self.device)
            self._forward(step, False, m, out)
            torch.cuda.current_stream(self.device).synchronize()
            graph = torch.cuda.CUDAGraph()
            before = getattr(kernels, "launches", 0)
            with torch.cuda.graph(graph, pool=self._graph_pool):
                self._forward(step, False, m, out)
            if hasattr(kernels, "launches"):
                captured, kernels.launches = kernels.launches - before, before   # recorded, not run
            else:
                captured = 0
            self._graph_pool = self._graph_pool or graph.pool()
            self._graphs[key] = (graph, out, captured)
            if any(e.from_last for e in entries):      # captured while the step before was still in flight
                self._captured_ahead.add(key)
            return out, [row_of[i] for i in wanted]
        graph, out, captured = self._graphs[key]
        graph.replay()
        self.graph_steps += 1
        self.mixed_graph_steps += bool(portions)
        self._graph_launches += captured
        return out, [row_of[i] for i in wanted]

    def _commit(self, inflight: "_Inflight") -> list[TokenDelta]:
        """Waits for a launched step and books its tokens: appended, checked for a finish, reported."""
        if inflight.done is not None:
            inflight.done.synchronize()
        self._check_kernels()
        tokens = inflight.host.tolist() if inflight.host is not None else []
        if inflight.pick is not None:
            tokens = [tokens[i] for i in inflight.pick]
        for request, chosen, ids, top in inflight.prompt:   # before any delta: a prompt's last piece and its first token
            acc = self._prompt_lp.get(request)             # come from the same step
            if acc is not None:
                acc.token += chosen.tolist()
                acc.top_ids += ids.tolist()
                acc.top += top.tolist()
        lps = [t.tolist() for t in inflight.logprobs] if inflight.logprobs is not None else None
        deltas = []
        for j, (row, token) in enumerate(zip(inflight.sampled, tokens)):
            request = row.request
            request.pending -= 1
            if request.status is Status.FINISHED:          # it stopped a step ago; this row was already in flight
                if request.pending == 0 and request.slot >= 0:
                    self.built.cache.release(request.slot)
                    request.slot = -1
                continue
            request.tokens.append(int(token))
            cached = None
            if request.status is not Status.RUNNING:
                self.scheduler.finished_prefill(request)
                if request.generated == 1:                 # its first token, not a return from preemption
                    cached = request.cached
                for sibling in self._siblings.pop(request, []):
                    self.scheduler.add(sibling)
            reason = self._finish_reason(request, int(token))
            if reason:
                self.scheduler.finish(request, reason, release=request.pending == 0)
                self._retire(request)
            k = request.params.logprobs
            own = None if k is None or lps is None else Logprobs([lps[0][j]], [lps[1][j][:k]], [lps[2][j][:k]])
            deltas.append(TokenDelta(request.rid, [int(token)], request.index, own, self._prompt_lp.pop(request, None),
                                     reason, cached))
        return deltas

    def _check_kernels(self) -> None:
        """Every wait inside the kernels is bounded; one that gave up left a code in a word of host memory, and what
        its kernel wrote is not to be trusted. Read here, after a step's completion event and before any of its
        tokens is handed out: the engine stops with the reason and refuses further work, as the reference stops when
        a step's commit fails (core/holon/core/engine.py:498-499, 607-612)."""
        status = getattr(self.built.ctx.kernels, "status", None)
        code = status() if status is not None else 0
        if code:
            self._stopped = (f"a bounded wait inside a kernel gave up (status {code:#010x}: place {code >> 28}, "
                             f"block {(code & 0x0FFFFFFF) - 1}); the step's results were dropped")
            self._inflight = None
            raise RuntimeError(f"the engine stopped: {self._stopped}")

    def _retire(self, request: Request) -> None:
        live = self.requests.get(request.rid)
        if live is not None and request in live:
            live.remove(request)
            if not live:
                del self.requests[request.rid]

    def _finish_reason(self, request: Request, token: int) -> str | None:
        p = request.params
        if (token in self.eos and not p.ignore_eos) or token in p.stop_token_ids:
            return "stop"
        if (p.max_tokens is not None and request.generated >= p.max_tokens) \
                or len(request.tokens) >= self.config.max_model_len:
            return "length"
        return None

    # ------------------------------------------------------------------ whole prompts
    def generate(self, prompts: Sequence[Sequence[int]], params: SamplingParams | Sequence[SamplingParams] | None = None
                 ) -> list[list[int]]:
        """The generated token ids of every prompt (host lists in, host lists out), in the prompts' order."""
        many = isinstance(params, (list, tuple))
        if any(p is not None and p.n != 1 for p in (params if many else [params])):
            raise ValueError("generate() returns one sequence per prompt; step() streams n > 1")
        rids = [self.add(p, params[i] if many else params) for i, p in enumerate(prompts)]
        out: dict[str, list[int]] = {rid: [] for rid in rids}
        while any(rid in self.requests for rid in rids):
            for delta in self.step():
                if delta.rid in out:
                    out[delta.rid].extend(delta.token_ids)
        if not self.requests:
            self.drain()                                   # (a last wasted row may still be in flight)
        return [out[rid] for rid in rids]

    def launches(self) -> int:
        """Kernels of this package launched so far: the ones enqueued directly plus, for every graph replay, the
        ones its capture recorded."""
        return getattr(self.built.ctx.kernels, "launches", 0) + self._graph_launches

    def stats(self) -> dict[str, int]:
        s, p = self.scheduler, self.built.cache.prefix
        return {"waiting": len(s.waiting), "running": len(s.running), "preemptions": s.preemptions,
                "mixed_steps": s.mixed_steps, "steps": self.steps, "graph_steps": self.graph_steps,
                "mixed_graph_steps": self.mixed_graph_steps,
                "graphs": len(self._graphs), "free_tokens": self.built.cache.free_tokens(),
                "prefix_hit_tokens": p.hits if p is not None else 0, "prefix_query_tokens": p.queries if p is not None else 0}

    def memory_report(self) -> str:
        """One line: what the weights, the largest step's activations, the graphs' pool and the cache pools take of
        the device's memory, and what is left (measured when the engine was built)."""
        return self.built.memory.line()

    def close(self) -> None:
        for rid in list(self.requests):
            self.abort(rid)
        if not self._stopped:
            self.drain()
        self._inflight = None
        self._graphs.clear()
