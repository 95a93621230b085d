"""From a weight source to a runnable model with its cache and step function
(core/holon/core/engine.py:143-282 without plugins, ledger profiling and prefix cache)."""
from __future__ import annotations

import dataclasses

import torch

from ..cache import CacheManager
from ..config.registry import resolve_architecture
from ..parts import BuildContext, Model
from ..weights import load_weights
from .runner import Runner

TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


@dataclasses.dataclass
class Built:
    config: object                # the architecture's typed configuration
    model: Model
    cache: CacheManager
    runner: Runner
    ctx: BuildContext
    weight_bytes: int


def build(source, *, dtype: str, device, kernels=None, page_size: int, max_seqs: int, max_model_len: int,
          max_step_tokens: int, state_memory: int | None = None, pages: int | None = None,
          memory_fraction: float = 0.9, prefix_cache: bool = False) -> Built:
    """`kernels=None` loads the compiled CUDA kernels and fails if they cannot be had. With neither `state_memory`
    nor `pages` the cache takes `memory_fraction` of the device memory left after the weights, less room for the
    largest step's activations."""
    device = torch.device(device)
    if kernels is None:
        from ..kernels import load_kernels
        kernels = load_kernels(device)
    tdtype = TORCH_DTYPES[dtype]
    raw = source.config()
    arch = resolve_architecture(raw)
    config = arch.parse(raw)
    spec = arch.recipe(config)
    ctx = BuildContext(device, tdtype, kernels, max_positions=max_model_len, max_step_tokens=max_step_tokens)
    model = Model(spec, ctx)
    weight_bytes = load_weights(model, spec, source.tensors(), tdtype, device)
    if state_memory is None and pages is None:
        free, _ = torch.cuda.mem_get_info(device)
        # room for the largest step's activations: a few tensors of the widest layer product per token, the 32-bit
        # stream, and logits for as many rows as can sample in one step
        widest = max([p.shape[0] for name, p in model.params() if p.kind == "matrix" and not name.startswith("head.")]
                     + [spec.hidden])
        activations = max_step_tokens * (widest * 3 + spec.hidden * 8) * 4 + min(max_step_tokens, max_seqs) * spec.vocab * 8
        state_memory = int(free * memory_fraction) - activations
    cache = CacheManager(model.entries, page_size, max_seqs, max_model_len, tdtype, device,
                         state_memory=state_memory, pages=pages, prefix_cache=prefix_cache)
    return Built(config, model, cache, Runner(model, cache, ctx, max_step_tokens), ctx, weight_bytes)
