"""Per-request sampling settings; names, defaults and meanings are the reference's `SamplingParams`
(core/holon/api/batch.py:45-61). Penalties are refused as they are there (core/holon/core/engine.py:346-347);
`logprobs` and `prompt_logprobs` ask for the top-k log-probabilities of generated and of prompt tokens."""
from __future__ import annotations

import dataclasses

SEED_MASK = 2 ** 63 - 1


@dataclasses.dataclass
class SamplingParams:
    temperature: float = 1.0                 # 0: greedy (arg max)
    top_p: float = 1.0                       # keep the smallest set of most likely tokens whose mass reaches top_p
    top_k: int = 0                           # keep the k most likely tokens (0: off)
    min_p: float = 0.0                       # drop tokens less likely than min_p × the most likely one
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    n: int = 1
    max_tokens: int | None = None
    ignore_eos: bool = False
    stop_token_ids: tuple[int, ...] = ()
    seed: int | None = None                  # None: the engine draws one
    logprobs: int | None = None              # top-k log-probabilities per generated token (0: the token's own alone)
    prompt_logprobs: int | None = None       # and per prompt token

    def validate(self) -> None:
        if (self.presence_penalty, self.frequency_penalty, self.repetition_penalty) != (0.0, 0.0, 1.0):
            raise NotImplementedError("presence, frequency and repetition penalties are not implemented")
        for name in ("logprobs", "prompt_logprobs"):
            k = getattr(self, name)
            if k is not None and (not isinstance(k, int) or k < 0):
                raise ValueError(f"SamplingParams.{name} must be None or a count >= 0, got {k!r}")
        if self.n < 1:
            raise ValueError("SamplingParams.n must be >= 1")
        if self.temperature < 0 or not 0 < self.top_p <= 1 or self.top_k < 0 or not 0 <= self.min_p <= 1:
            raise ValueError(f"SamplingParams out of range: {self}")
        if self.max_tokens is not None and self.max_tokens < 1:
            raise ValueError("SamplingParams.max_tokens must be >= 1")

    @property
    def filtered(self) -> bool:
        return self.temperature > 0 and (self.top_k > 0 or self.top_p < 1 or self.min_p > 0)


def sequence_seed(seed: int, index: int) -> int:
    """The seed of sequence `index` of a request with `n` > 1: sequence 0 keeps the request's seed, the others get
    it mixed with their index by splitmix64 (core/holon/api/batch.py:64-77)."""
    base = seed & SEED_MASK
    if index == 0:
        return base
    m = 0xFFFFFFFFFFFFFFFF
    x = (base + index + 0x9E3779B97F4A7C15) & m
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & m
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & m
    return (x ^ (x >> 31)) & SEED_MASK
