"""Which requests run in the next step, and with how many tokens each.

First come, first served. Requests are ranked: running ones (oldest first), then waiting ones (queue order).
Without mixing (`chunk_with_decode` 0) a step prefills while a waiting request can be admitted, in portions under
the token budget `max_step_tokens`, and otherwise decodes every running request. With mixing (C > 0) a step carries
the running requests' decode rows first and then prompt portions of at most C tokens in all; a step with nothing to
decode prefills up to the full budget (core/holon/core/sched.py:1-44, 106-187).

When pages run out: the asker may take them from requests ranked below it. The lowest-ranked admitted request is
preempted, again and again, while that can make room; a preempted request gives back everything, keeps its tokens
(prompt and generated), goes to the front of the waiting queue and is computed again from its first token when it is
admitted anew. If nothing below can make room, a running request preempts itself and a waiting one ends the step's
prefill (sched.py:189-207). Sampling is a function of (seed, position), so the tokens do not change. The pools hold
at least one request of the longest length, so the top-ranked request always runs: every step makes progress.
"""
from __future__ import annotations

import collections
import dataclasses
import enum

from ..sampling.params import SamplingParams


class Status(enum.Enum):
    WAITING = 0
    RUNNING = 1
    PREEMPTED = 2
    FINISHED = 3


@dataclasses.dataclass(eq=False)
class Request:
    rid: str
    tokens: list[int]                       # prompt, then generated tokens
    prompt_len: int
    params: SamplingParams
    seed: int = 0
    index: int = 0                          # which of its request's `n` sequences this is
    cached: int | None = None               # tokens the prefix cache served when it was first admitted
    slot: int = -1
    computed: int = 0                       # tokens whose keys and values the cache holds (or is being given)
    pending: int = 0                        # tokens sampled by steps in flight, not yet read back
    status: Status = Status.WAITING
    finish_reason: str | None = None

    @property
    def generated(self) -> int:
        return len(self.tokens) - self.prompt_len


@dataclasses.dataclass
class Row:
    request: Request
    n_tokens: int
    samples: bool                           # the row ends at the request's last token: its logits are sampled


class Scheduler:
    def __init__(self, cache, max_step_tokens: int, max_model_len: int, chunk_with_decode: int = 0) -> None:
        self.cache, self.max_step_tokens, self.max_model_len = cache, max_step_tokens, max_model_len
        self.chunk_with_decode = chunk_with_decode
        self.waiting: collections.deque[Request] = collections.deque()
        self.running: list[Request] = []
        self.preemptions = 0
        self.mixed_steps = 0

    def add(self, request: Request, front: bool = False) -> None:
        request.status = Status.WAITING
        (self.waiting.appendleft if front else self.waiting.append)(request)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ one step's rows
    def schedule(self) -> list[Row] | None:
        """The next step's rows, decode rows first; None if nothing can run."""
        cap = self.chunk_with_decode
        if not cap:
            rows = self._prefill(self.max_step_tokens) or self._decode()
        else:
            rows = self._decode()
            if not rows:
                rows = self._prefill(self.max_step_tokens)
            else:
                chunks = self._prefill(min(cap, self.max_step_tokens - len(rows)))
                self.mixed_steps += bool(chunks)
                rows = rows + chunks
        return rows or None

    def _prefill(self, budget: int) -> list[Row]:
        rows = []
        for request in list(self.waiting):
            if budget <= 0:
                break
            if request.slot < 0 and not self._fit(request, None):
                break
            n = min(len(request.tokens) - request.computed, budget)
            chunk = getattr(self.cache, "chunk", 1)
            if chunk > 1 and request.computed + n < len(request.tokens):
                n -= (request.computed + n) % chunk          # a portion that does not end the prompt ends on a multiple
                if n <= 0:                                   # (the budget left is too small for one chunk: next step)
                    break
            if not self._fit(request, request.computed + n):
                break
            rows.append(Row(request, n, request.computed + n == len(request.tokens)))
            budget -= n
        return rows

    def _decode(self) -> list[Row]:
        rows = []
        for request in list(self.running):
            if request.status is not Status.RUNNING or self.at_limit(request):    # preempted by a row above it
                continue
            need = request.computed + 1
            if need <= self.cache.capacity(request.slot) or self._fit(request, need):
                rows.append(Row(request, 1, True))
            else:
                self._preempt(request)
        return rows

    def at_limit(self, request: Request) -> bool:
        """Counting the tokens still in flight: a request at its limit is not scheduled again; its commit ends it."""
        m, length = request.params.max_tokens, len(request.tokens) + request.pending
        return length >= self.max_model_len or (m is not None and length - request.prompt_len >= m)

    # ------------------------------------------------------------------ room
    def _fit(self, request: Request, tokens: int | None) -> bool:
        """Admit `request` (tokens None) or reserve pages so that it holds `tokens` positions, preempting
        lower-ranked admitted requests, lowest first, while releasing them can make room."""
        while True:
            if tokens is None:
                # (prompt logprobs need every prompt position computed: such a request starts on no cached prefix)
                wants_all = request.index == 0 and request.params.prompt_logprobs is not None
                slot = self.cache.admit(None if wants_all else request.tokens)
                if slot is not None:
                    request.slot, request.computed = slot, int(self.cache.computed[slot])
                    if request.cached is None:
                        request.cached = request.computed            # what the prefix cache served at its first admission
                    return True
            elif self.cache.reserve(request.slot, tokens):
                return True
            ranked = self.running + list(self.waiting)
            below = [r for r in ranked[ranked.index(request) + 1:] if r.slot >= 0]
            if not below:
                return False
            if tokens is not None and not self.cache.could_fit(request.slot, tokens, [r.slot for r in below]):
                return False
            self._preempt(below[-1])

    def _preempt(self, request: Request) -> None:
        self.cache.release(request.slot)
        request.slot, request.computed = -1, 0
        self.preemptions += 1
        if request.status is Status.RUNNING:          # back to the head of the queue, before requests never run
            self.running.remove(request)
            self.waiting.appendleft(request)
            request.status = Status.PREEMPTED

    # ------------------------------------------------------------------ what the engine reports back
    def computed(self, row: Row) -> None:
        row.request.computed += row.n_tokens

    def finished_prefill(self, request: Request) -> None:
        self.waiting.remove(request)
        request.status = Status.RUNNING
        self.running.append(request)

    def finish(self, request: Request, reason: str, release: bool = True) -> None:
        """`release=False`: a row of this request is still in flight; whoever commits it gives the slot back."""
        (self.running if request.status is Status.RUNNING else self.waiting).remove(request)
        if release and request.slot >= 0:
            self.cache.release(request.slot)
            request.slot = -1
        request.status, request.finish_reason = Status.FINISHED, reason
