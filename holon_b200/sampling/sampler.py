"""Turns a step's logits rows into tokens with the sampling kernel.

Greedy rows take the arg max. Sampled rows: softmax(logits / temperature), optionally filtered (top-k, then top-p
over the renormalised rest, then min-p), and one token drawn by inverse CDF with a uniform that is a hash of
(seed, position of the token being drawn). There is no generator state, so a request draws the same tokens whatever
else is in the batch and however often it is preempted (std/holon_std/sampling/sampler.py:24-61, 128-152;
std/holon_std/sampling/reference.py:13-30). One difference: the reference draws filtered rows in order of
descending logit, this sampler draws every row in vocabulary order; the distribution is the same, the token picked
by a given uniform is not.
"""
from __future__ import annotations

import numpy as np
import torch


def sampling_arrays(rows) -> dict[str, np.ndarray]:
    """int32 arrays for the upload buffer from (params, seed, position) per logits row; floats keep their bits."""
    n = len(rows)
    temperature, top_p, min_p = (np.zeros(n, dtype=np.float32) for _ in range(3))
    top_k, lo, hi, position = (np.zeros(n, dtype=np.int64) for _ in range(4))
    for i, (p, seed, pos) in enumerate(rows):
        temperature[i], top_p[i], min_p[i], top_k[i] = p.temperature, p.top_p, p.min_p, p.top_k
        lo[i], hi[i], position[i] = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF, pos
    as_i32 = lambda a: a.astype(np.uint32).view(np.int32)             # noqa: E731
    return {"temperature": temperature.view(np.int32), "top_p": top_p.view(np.int32), "min_p": min_p.view(np.int32),
            "top_k": top_k.astype(np.int32), "seed_lo": as_i32(lo), "seed_hi": as_i32(hi),
            "sample_position": position.astype(np.int32)}


class Sampler:
    def __init__(self, kernels, device) -> None:
        self.kernels, self.device = kernels, torch.device(device)

    def sample(self, logits: torch.Tensor, dev: dict[str, torch.Tensor], filtered: bool,
               out: torch.Tensor | None = None) -> torch.Tensor:
        """`dev`: the device views of `sampling_arrays`. Returns int32 tokens [rows]."""
        tokens = out if out is not None else torch.empty(logits.shape[0], dtype=torch.int32, device=self.device)
        f32 = lambda name: dev[name].view(torch.float32)             # noqa: E731
        self.kernels.sample(tokens, logits, f32("temperature"), dev["top_k"], f32("top_p"), f32("min_p"),
                            dev["seed_lo"], dev["seed_hi"], dev["sample_position"], filtered)
        return tokens

    def logprobs(self, logits: torch.Tensor, tokens: torch.Tensor, k: int):
        """Of the raw logits, before temperature and filters (std/holon_std/sampling/sampler.py:118-126): float32 [rows]
        log softmax(logits)[tokens], and the `k` most likely per row as int32 ids and float32 log-probabilities
        [rows, k], ranked, equal logits by ascending id."""
        r = logits.shape[0]
        chosen = torch.empty(r, dtype=torch.float32, device=self.device)
        top_ids = torch.empty((r, k), dtype=torch.int32, device=self.device)
        top = torch.empty((r, k), dtype=torch.float32, device=self.device)
        self.kernels.logprobs(chosen, top_ids, top, logits, tokens)
        return chosen, top_ids, top
