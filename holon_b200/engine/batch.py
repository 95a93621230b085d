"""A step's batch: what the caller gives (`StepEntry`) and what the model sees on the device (`StepContext`).

The layout is the reference's: flat and token-major, rows marked by `query_start`, with a block table and write
indices per cache group (core/holon/api/batch.py:123-152; core/holon/api/state.py:56-68). A row is a request's
next tokens; a prompt portion and a single decoded token differ only in their length.
"""
from __future__ import annotations

import dataclasses
from collections.abc import Sequence

import numpy as np
import torch

from ..parts.model import LayerCache


@dataclasses.dataclass
class StepEntry:
    """Request in slot `slot` brings `tokens`, which take positions `start`, `start + 1`, …; `want` lists the places
    among these tokens whose logits the caller asks for (it may be empty)."""

    slot: int
    tokens: Sequence[int]
    start: int
    want: Sequence[int] = ()
    from_last: bool = False        # its one token is the one this request sampled last, still on the device


class Rows:
    """The step's rows as attention needs them. Device: `row_slot` [B], `query_start` [B+1], `kv_len` [B] (tokens a
    row holds after this step), all int32. Host: the same as numpy, and the counts kernels size their grids with.
    Rows that bring one token come first (`n_decode` of them)."""

    __slots__ = ("row_slot", "query_start", "kv_len", "n_rows", "n_tokens", "n_decode", "max_q", "max_kv",
                 "host_query_start", "host_kv_len", "plan")

    def __init__(self, row_slot, query_start, kv_len, n_rows, n_tokens, n_decode, max_q, max_kv,
                 host_query_start=None, host_kv_len=None) -> None:
        self.row_slot, self.query_start, self.kv_len = row_slot, query_start, kv_len
        self.n_rows, self.n_tokens, self.n_decode, self.max_q, self.max_kv = n_rows, n_tokens, n_decode, max_q, max_kv
        self.host_query_start, self.host_kv_len = host_query_start, host_kv_len
        self.plan: dict = {}                           # what the kernel table worked out for these rows, for the next layer


class GroupStep:
    """One cache group's part of a step: the device block table and, per token, page · page_size + offset."""

    __slots__ = ("block_table", "write_index", "page_size")

    def __init__(self, block_table, write_index, page_size) -> None:
        self.block_table, self.write_index, self.page_size = block_table, write_index, page_size


class StepContext:
    def __init__(self, token_ids, positions, logits_index, rows: Rows, groups: list[GroupStep], cache) -> None:
        self.token_ids, self.positions, self.logits_index, self.rows = token_ids, positions, logits_index, rows
        self.groups, self._cache = groups, cache
        self.extra: dict = {}
        self.link = None             # parts.base.Link: a block's offer to the product that ends its mixer or feed-forward
        self.from_last = None        # int32 [rows]: 1 where the row's token is fed from the device
        self.offset_of: dict = {}    # host: entry index -> offset of its first token among the step's tokens

    def layer_cache(self, run) -> LayerCache:
        c = self._cache
        group = c.group_of_entry.get(run.cache)
        slots = {name: t for (entry, name), t in c.slot_states.items() if entry == run.cache}
        if group is None:
            return LayerCache(None, None, run.fills, slots)
        return LayerCache(c.kv_of_entry[run.cache], self.groups[group.index], run.fills, slots)


class Uploader:
    """One page-locked host buffer and one device buffer of int32: a step's small arrays are laid out one after the
    other on the host and go over in a single copy (core/holon/core/inputs.py:24-87). Two host buffers alternate, and
    a buffer is written again only after the copy that read it last has finished."""

    ALIGN = 4                                     # int32 elements: every array starts on a 16-byte boundary

    def __init__(self, capacity: int, device) -> None:
        self.device = torch.device(device)
        cuda = self.device.type == "cuda"
        self._host = [torch.zeros(capacity, dtype=torch.int32) for _ in range(2)]
        if cuda:
            self._host = [h.pin_memory() for h in self._host]
        self._np = [h.numpy() for h in self._host]
        self._events = [torch.cuda.Event() if cuda else None for _ in range(2)]
        self._used = [False, False]
        self.dev = torch.zeros(capacity, dtype=torch.int32, device=self.device)
        self._which, self._at, self._views = 0, 0, {}
        self.bytes_last = 0

    def begin(self) -> None:
        self._which ^= 1
        if self._used[self._which] and self._events[self._which] is not None:
            self._events[self._which].synchronize()
        self._at, self._views = 0, {}

    def put(self, name: str, array: np.ndarray) -> None:
        n = int(array.shape[0])
        if self._at + n > self.dev.shape[0]:
            raise ValueError(f"a step's arrays need more than the {self.dev.shape[0]} int32 the upload buffer holds")
        self._np[self._which][self._at:self._at + n] = array
        self._views[name] = (self._at, n)
        self._at = -(-(self._at + n) // self.ALIGN) * self.ALIGN

    def end(self) -> dict[str, torch.Tensor]:
        w, n = self._which, self._at
        if n:
            self.dev[:n].copy_(self._host[w][:n], non_blocking=True)
        if self._events[w] is not None:
            self._events[w].record()
            self._used[w] = True
        self.bytes_last = n * 4
        return {name: self.dev[a:a + m] for name, (a, m) in self._views.items()}
