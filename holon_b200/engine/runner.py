"""The step function: a batch of (request, its next tokens) in, logits at the wanted places out.

It runs only the tokens it is given, as one batch, reading everything earlier from the cache
(core/holon/core/executor.py:357-430, 497-564). The caller (the scheduler's engine, or the replay tool) has
admitted the requests and reserved their pages; the step checks that and fails before it touches the device.
"""
from __future__ import annotations

from collections.abc import Sequence

import numpy as np
import torch

from .batch import GroupStep, Rows, StepContext, StepEntry, Uploader


class StepError(ValueError):
    """A batch that cannot run: tokens out of order, pages not reserved, too many tokens."""


class Runner:
    def __init__(self, model, cache, build_ctx, max_step_tokens: int) -> None:
        self.model, self.cache, self.ctx = model, cache, build_ctx
        self.device, self.max_step_tokens = build_ctx.device, max_step_tokens
        s, t, g = cache.max_seqs + 1, max_step_tokens, len(cache.groups)
        tables = sum(s * (group.max_pages + 1) + 8 for group in cache.groups)     # every block-table row changed at once
        self.uploader = Uploader(t * (3 + g) + 16 * s + 64 + tables, self.device)
        self.vocab = model.spec.vocab

    # ------------------------------------------------------------------ host half
    def check(self, entries: Sequence[StepEntry]) -> None:
        c, seen, total = self.cache, set(), 0
        if not entries:
            raise StepError("a step needs at least one entry")
        for e in entries:
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"slot {e.slot}: an entry brings no tokens")
            if e.slot not in c.live:
                raise StepError(f"slot {e.slot} is not admitted")
            if e.slot in seen:
                raise StepError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            if e.start != int(c.computed[e.slot]):
                raise StepError(f"slot {e.slot}: tokens start at {e.start}, the cache holds {int(c.computed[e.slot])}")
            if e.start + n > c.capacity(e.slot):
                raise StepError(f"slot {e.slot}: pages for {e.start + n} tokens are not reserved "
                                f"(capacity {c.capacity(e.slot)})")
            if any(not 0 <= w < n for w in e.want):
                raise StepError(f"slot {e.slot}: wanted places {list(e.want)} are outside its {n} tokens")
            if e.from_last and n != 1:
                raise StepError(f"slot {e.slot}: only a single token can be fed from the device")
            if any(not 0 <= t < self.vocab for t in e.tokens):
                raise StepError(f"slot {e.slot}: a token id is outside the vocabulary of {self.vocab}")
            total += n
        if total > self.max_step_tokens:
            raise StepError(f"{total} tokens in one step; max_step_tokens is {self.max_step_tokens}")

    def context(self, entries: Sequence[StepEntry], pad_rows: int | None = None, extra=None) -> StepContext:
        """Lays the batch out (rows of one token first), uploads it in one copy and returns the device-side view.
        `pad_rows` (not None: the step runs as a CUDA graph): so many rows of one token each for the padding slot
        follow the entries' one-token rows, and logits are taken at the last token of every row, padding included,
        so that the layout and the work depend on the counts alone (one-token rows with padding, rows of several
        tokens, tokens), not on the entries.
        `extra`: {name: int32 array} uploaded alongside; the device views land in `StepContext.extra`."""
        c = self.cache
        order = sorted(range(len(entries)), key=lambda i: len(entries[i].tokens) != 1)       # stable
        counts = [len(entries[i].tokens) for i in order]
        n_decode = sum(1 for n in counts if n == 1)
        bucket = pad_rows is not None
        pad_rows = pad_rows or 0
        if pad_rows:
            counts[n_decode:n_decode] = [1] * pad_rows
        b = len(counts)
        query_start = np.zeros(b + 1, dtype=np.int32)
        np.cumsum(counts, out=query_start[1:])
        t = int(query_start[-1])
        token_ids, positions = np.zeros(t, dtype=np.int32), np.zeros(t, dtype=np.int32)
        row_slot, kv_len = np.full(b, c.padding_slot, dtype=np.int32), np.ones(b, dtype=np.int32)
        token_slot = np.full(t, c.padding_slot, dtype=np.int32)
        from_last = np.zeros(b, dtype=np.int32)
        offset_of = {}
        rows = list(range(n_decode)) + list(range(n_decode + pad_rows, b))
        for r, i in zip(rows, order):
            e, a, n = entries[i], int(query_start[r]), counts[r]
            token_ids[a:a + n] = e.tokens
            positions[a:a + n] = np.arange(e.start, e.start + n)
            token_slot[a:a + n] = e.slot
            row_slot[r], kv_len[r] = e.slot, e.start + n
            from_last[r] = int(e.from_last)
            offset_of[i] = a
        if bucket:
            logits_index = query_start[1:] - 1
        else:
            logits_index = np.array([offset_of[i] + w for i, e in enumerate(entries) for w in e.want], dtype=np.int32)
        up = self.uploader
        up.begin()
        up.put("token_ids", token_ids)
        up.put("positions", positions)
        up.put("query_start", query_start)
        up.put("row_slot", row_slot)
        up.put("kv_len", kv_len)
        up.put("logits_index", logits_index)
        up.put("from_last", from_last)
        for g in c.groups:
            up.put(f"write_index.{g.index}", g.write_index(token_slot, positions).astype(np.int32))
        for name, array in (extra or {}).items():
            up.put(name, array)
        changed = []
        for g in c.groups:                            # block-table rows that changed, behind everything a graph reads
            slots, table_rows = g.take_dirty()        # (copies: the host table may change before the upload is read)
            if len(slots):
                up.put(f"table_slots.{g.index}", slots)
                up.put(f"table_rows.{g.index}", table_rows.reshape(-1))
                changed.append(g)
        dev = up.end()
        for g in changed:
            self.ctx.kernels.scatter_rows(g.table_device, dev[f"table_slots.{g.index}"], dev[f"table_rows.{g.index}"])
        rows_ = Rows(dev["row_slot"], dev["query_start"], dev["kv_len"], b, t, n_decode + pad_rows,
                     max(counts), int(kv_len.max()), query_start, kv_len)
        groups = [GroupStep(g.table_device, dev[f"write_index.{g.index}"], g.page_size) for g in c.groups]
        step = StepContext(dev["token_ids"], dev["positions"], dev["logits_index"], rows_, groups, c)
        step.extra = {name: dev[name] for name in (extra or {})}
        step.from_last = dev["from_last"]
        step.offset_of = offset_of                    # entry index -> where its tokens start among the step's
        return step

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor | None:
        """Logits [wanted, vocab] in 32-bit, in the order of the entries and of each entry's `want`; None when
        nothing is wanted. Afterwards the cache holds the step's tokens."""
        self.check(entries)
        step = self.context(entries)
        logits = self.model.forward(step)
        self.commit(entries)
        return logits

    def commit(self, entries: Sequence[StepEntry]) -> None:
        for e in entries:
            self.cache.advance(e.slot, e.start + len(e.tokens))
