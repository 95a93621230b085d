"""The engine a user calls: requests in, tokens out.

`Engine(EngineConfig(model=...)).generate(prompts, params)` returns the generated token ids of each prompt;
`add` / `step` / `has_work` / `abort` / `stats` / `close` drive it by hand. Names and meanings follow the reference
(core/holon/core/engine.py:332-376, 461-524, 702-709). Every step runs at depth 0: schedule, run, sample, read the
tokens back, commit.
"""
from __future__ import annotations

import dataclasses
import secrets
from collections.abc import Sequence

import numpy as np
import torch

from ..config.engine import EngineConfig
from ..sampling import Sampler, SamplingParams, sampling_arrays, sequence_seed
from ..sampling.params import SEED_MASK
from ..weights import SafetensorsSource
from .batch import StepEntry
from .build import build
from .scheduler import Request, Row, Scheduler

GRAPH_BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)


@dataclasses.dataclass
class TokenDelta:
    """What one step added to one request (core/holon/api/frontend.py:17-52)."""

    rid: str
    token_ids: list[int]
    index: int                               # how many tokens the request had generated before these
    finish_reason: str | None = None         # "stop" | "length" | "abort" | None


class Engine:
    def __init__(self, config: EngineConfig, source=None, kernels=None) -> None:
        """`source`: a weight source in place of the folder `config.model` (random weights, for one);
        `kernels`: a kernel table in place of the compiled CUDA kernels (tests on a machine without a GPU)."""
        self.config = config
        source = source or SafetensorsSource(config.model)
        self.built = build(source, dtype=config.dtype, device=config.device, kernels=kernels,
                           page_size=config.page_size, max_seqs=config.max_seqs, max_model_len=config.max_model_len,
                           max_step_tokens=config.max_step_tokens, state_memory=config.state_memory,
                           memory_fraction=config.memory_fraction)
        b = self.built
        self.device = b.ctx.device
        self.eos = frozenset(source.eos_token_ids())
        self.scheduler = Scheduler(b.cache, config.max_step_tokens, config.max_model_len, config.chunk_with_decode)
        self.sampler = Sampler(b.ctx.kernels, self.device)
        self.requests: dict[str, Request] = {}
        self._base_seed = config.seed if config.seed is not None else secrets.randbits(63)
        self._added = 0
        self._graphs: dict[int, tuple] = {}
        self._graph_pool = None
        self._use_graphs = config.cuda_graphs and self.device.type == "cuda"
        self._buckets = tuple(x for x in GRAPH_BUCKETS if x <= config.max_seqs)
        self._host_tokens = torch.zeros(config.max_step_tokens, dtype=torch.int32)
        if self.device.type == "cuda":
            self._host_tokens = self._host_tokens.pin_memory()
        self.steps = self.graph_steps = self._graph_launches = 0
        self.h2d_bytes = self.d2h_bytes = 0

    # ------------------------------------------------------------------ requests
    def add(self, token_ids: Sequence[int], params: SamplingParams | None = None, rid: str | None = None) -> str:
        params = params or SamplingParams()
        params.validate()
        if params.n != 1:
            raise NotImplementedError("n > 1: add the prompt n times with seeds from sampling.sequence_seed")
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
        seed = (params.seed if params.seed is not None else sequence_seed(self._base_seed, self._added + 1)) & SEED_MASK
        self._added += 1
        self.requests[rid] = request = Request(rid, tokens, len(tokens), params, seed)
        self.scheduler.add(request)
        return rid

    def abort(self, rid: str) -> TokenDelta | None:
        request = self.requests.pop(rid, None)
        if request is None:
            return None
        self.scheduler.finish(request, "abort")
        return TokenDelta(rid, [], request.generated, "abort")

    def has_work(self) -> bool:
        return self.scheduler.has_work()

    # ------------------------------------------------------------------ one step
    def step(self) -> list[TokenDelta]:
        rows = self.scheduler.schedule()
        if rows is None:
            if self.has_work():
                raise RuntimeError("the scheduler made no progress with requests pending")
            return []
        entries = [StepEntry(r.request.slot, r.request.tokens[r.request.computed:r.request.computed + r.n_tokens],
                             r.request.computed, (r.n_tokens - 1,) if r.samples else ()) for r in rows]
        sampled = [r for r in rows if r.samples]
        tokens = self._run(entries, sampled) if sampled else self._run_quiet(entries)
        self.steps += 1
        for r in rows:
            self.scheduler.computed(r)
        return [self._commit(r, t) for r, t in zip(sampled, tokens)]

    def _run_quiet(self, entries) -> list[int]:
        """A step in which every row stops short of its prompt's end: nothing is sampled, the head is skipped."""
        runner = self.built.runner
        runner.check(entries)
        runner.model.forward(runner.context(entries))
        runner.commit(entries)
        self.h2d_bytes += runner.uploader.bytes_last
        return []

    def _run(self, entries, sampled: list[Row]) -> list[int]:
        runner, n = self.built.runner, len(sampled)
        runner.check(entries)
        arrays = sampling_arrays([(r.request.params, r.request.seed, r.request.computed + r.n_tokens)
                                  for r in sampled])
        filtered = any(r.request.params.filtered for r in sampled)
        decode_only = len(sampled) == len(entries) and all(len(e.tokens) == 1 for e in entries)
        if self._use_graphs and decode_only and not filtered and n <= (self._buckets[-1] if self._buckets else 0):
            tokens = self._replay(entries, arrays)
        else:
            step = runner.context(entries, extra=arrays)
            logits = runner.model.forward(step)
            tokens = self.sampler.sample(logits, step.extra, filtered)
        self.h2d_bytes += runner.uploader.bytes_last
        host = self._host_tokens[:n]
        host.copy_(tokens[:n], non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize() if self.device.type == "cuda" else None
        self.d2h_bytes += n * 4
        runner.commit(entries)
        return host.tolist()

    def _replay(self, entries, arrays) -> torch.Tensor:
        """A decode step through the CUDA graph of its batch-size bucket (core/holon/core/executor.py:316-344):
        rows are padded to the bucket with rows of the padding slot, which read and write the null page."""
        runner, n = self.built.runner, len(entries)
        bucket = next(b for b in self._buckets if b >= n)
        pad = bucket - n
        padded = {k: np.concatenate([v, np.zeros(pad, dtype=v.dtype)]) for k, v in arrays.items()}
        step = runner.context(entries, pad_rows=pad, extra=padded)
        if bucket not in self._graphs:
            step.rows.max_kv = self.config.max_model_len          # the captured launch must serve any length
            out = torch.empty(bucket, dtype=torch.int32, device=self.device)
            self.sampler.sample(runner.model.forward(step), step.extra, False, out)      # warm-up, not captured
            torch.cuda.current_stream(self.device).synchronize()
            graph, kernels = torch.cuda.CUDAGraph(), self.built.ctx.kernels
            before = kernels.launches
            with torch.cuda.graph(graph, pool=self._graph_pool):
                self.sampler.sample(runner.model.forward(step), step.extra, False, out)
            captured, kernels.launches = kernels.launches - before, before       # recorded, not run
            self._graph_pool = self._graph_pool or graph.pool()
            self._graphs[bucket] = (graph, out, captured)
        graph, out, captured = self._graphs[bucket]
        graph.replay()
        self.graph_steps += 1
        self._graph_launches += captured
        return out

    def _commit(self, row: Row, token: int) -> TokenDelta:
        request = row.request
        index = request.generated
        request.tokens.append(int(token))
        if request.status.name != "RUNNING":
            self.scheduler.finished_prefill(request)
        reason = self._finish_reason(request, int(token))
        if reason:
            self.scheduler.finish(request, reason)
            del self.requests[request.rid]
        return TokenDelta(request.rid, [int(token)], index, reason)

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
        rids = [self.add(p, params[i] if many else params) for i, p in enumerate(prompts)]
        out: dict[str, list[int]] = {rid: [] for rid in rids}
        while any(rid in self.requests for rid in rids):
            for delta in self.step():
                if delta.rid in out:
                    out[delta.rid].extend(delta.token_ids)
        return [out[rid] for rid in rids]

    def launches(self) -> int:
        """Kernels of this package launched so far: the ones enqueued directly plus, for every graph replay, the
        ones its capture recorded."""
        return getattr(self.built.ctx.kernels, "launches", 0) + self._graph_launches

    def stats(self) -> dict[str, int]:
        s = self.scheduler
        return {"waiting": len(s.waiting), "running": len(s.running), "preemptions": s.preemptions,
                "mixed_steps": s.mixed_steps, "steps": self.steps, "graph_steps": self.graph_steps,
                "graphs": len(self._graphs), "free_tokens": self.built.cache.free_tokens()}

    def close(self) -> None:
        for rid in list(self.requests):
            self.abort(rid)
        self._graphs.clear()
