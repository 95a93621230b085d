"""Engine settings. Field names and meanings follow the reference's `EngineConfig`
(core/holon/core/engine.py:61-100), one command-line flag per field; fields of features this engine does not have
(drafts, kernel pins and preferences, memory tiers, plugin options) are absent."""
from __future__ import annotations

import dataclasses

DTYPES = ("bfloat16", "float32")


def _setting(default, help: str):
    return dataclasses.field(default=default, metadata={"help": help})


@dataclasses.dataclass
class EngineConfig:
    model: str = dataclasses.field(metadata={"help": "model folder: config.json and *.safetensors"})
    device: str = _setting("cuda:0", "CUDA device to run on")
    dtype: str = _setting("bfloat16", "bfloat16: the serving kernels; float32: every product and sum in true 32-bit")
    page_size: int = _setting(64, "tokens per page of the key/value cache")
    max_seqs: int = _setting(64, "sequences served at once")
    max_model_len: int = _setting(8192, "prompt + generated tokens per request; the cache always holds one")
    max_step_tokens: int = _setting(4096, "tokens one step computes at most")
    chunk_with_decode: int = _setting(0, "prefill tokens a step with decode rows may also carry (0: none)")
    prefix_cache: bool = _setting(True, "share whole cache pages of equal prompt prefixes between requests")
    memory_fraction: float = _setting(0.9, "of the memory left after the weights, for the cache and activations")
    state_memory: int | None = _setting(None, "bytes for the cache pools; default: from memory_fraction")
    overlap: bool = _setting(True, "schedule step N while step N-1 runs (depth 1); off: depth 0")
    cuda_graphs: bool = _setting(True, "replay decode steps from CUDA graphs, per batch-size bucket")
    seed: int | None = _setting(None, "base seed for requests that bring none; default: drawn at start")

    def __post_init__(self) -> None:
        for name in ("page_size", "max_seqs", "max_model_len", "max_step_tokens"):
            if getattr(self, name) < 1:
                raise ValueError(f"EngineConfig.{name} must be >= 1")
        if self.chunk_with_decode < 0:
            raise ValueError("EngineConfig.chunk_with_decode must be >= 0")
        if self.dtype not in DTYPES:
            raise ValueError(f"EngineConfig.dtype must be one of {DTYPES}, not {self.dtype!r}")
        if self.chunk_with_decode and self.max_step_tokens < self.max_seqs + self.chunk_with_decode:
            raise ValueError("EngineConfig: mixed steps need max_step_tokens >= max_seqs + chunk_with_decode")
        if not 0 < self.memory_fraction <= 1:
            raise ValueError("EngineConfig.memory_fraction must be in (0, 1]")
