"""Sampling: per-request settings and the sampler that draws tokens from logits."""
from .params import SamplingParams, sequence_seed
from .sampler import Sampler, sampling_arrays

__all__ = ["Sampler", "SamplingParams", "sampling_arrays", "sequence_seed"]
