"""From a weight source to a runnable model with its cache and step function, and the account of the device's
memory that goes with it (core/holon/core/engine.py:143-282; the account: core/holon/core/executor.py:208-234)."""
from __future__ import annotations

import dataclasses
import math

import numpy as np
import torch

from ..cache import CacheManager
from ..config.registry import resolve_architecture
from ..parts import BuildContext, Model
from ..weights import load_weights
from .batch import StepEntry
from .runner import Runner

TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


@dataclasses.dataclass
class Memory:
    """Bytes of device memory, as found when the engine was built. `activations` and `graphs` are measured (the peak
    of a worst-case step, and of the largest step that is replayed from a graph) when the cache's size follows from
    `memory_fraction`; with a size given by the caller nothing is run and they are None."""

    weights: int
    cache: int
    activations: int | None
    graphs: int | None
    free_before: int | None                  # free on the device after the weights, before the cache pools
    free_after: int | None

    def line(self) -> str:
        gb = lambda b: "not measured" if b is None else f"{b / 2 ** 30:.2f} GiB"       # noqa: E731
        return (f"memory: weights {gb(self.weights)}, activations of the largest step {gb(self.activations)}, "
                f"graph pool {gb(self.graphs)}, cache pools {gb(self.cache)}, free {gb(self.free_after)}")


@dataclasses.dataclass
class Built:
    config: object                # the architecture's typed configuration
    model: Model
    cache: CacheManager
    runner: Runner
    ctx: BuildContext
    weight_bytes: int
    memory: Memory | None = None


def _peak_of(device, run) -> int:
    """Bytes `run()` needed at most beyond what was held before: what the allocator took from the device meanwhile
    (its own rounding and splitting of blocks included: that is what the cache pools must leave room for), and at
    least what it handed out (a small step may fit into blocks the allocator already holds)."""
    torch.cuda.synchronize(device)
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats(device)
    reserved, allocated = torch.cuda.memory_reserved(device), torch.cuda.memory_allocated(device)
    run()
    torch.cuda.synchronize(device)
    return max(0, torch.cuda.max_memory_reserved(device) - reserved, torch.cuda.max_memory_allocated(device) - allocated)


def _measure(model, ctx, entries, *, page_size: int, max_seqs: int, max_model_len: int, max_step_tokens: int,
             chunk_with_decode: int, dtype, device) -> tuple[int, int]:
    """The activation peaks of (1) the largest step the scheduler can make: `max_step_tokens` prompt tokens in as
    many rows as may end a prompt in one step, every row sampled; (2) the largest step replayed from a CUDA graph:
    one token for every sequence beside `chunk_with_decode` prompt tokens. Both run through the engine's own step
    function on pools just large enough to hold them, which are freed again (executor.py:208-234 does the same on
    minimum-size pools)."""
    from ..sampling import Sampler, SamplingParams, sampling_arrays
    rows = max(1, min(max_seqs, max_step_tokens))
    tokens = min(max_step_tokens, rows * (max_model_len - 1))
    ones = [1] * max(1, rows - bool(chunk_with_decode))
    portion = [min(chunk_with_decode, max_model_len - 1, max_step_tokens - len(ones))] if chunk_with_decode else []
    pages = max(math.ceil(max_model_len / page_size), rows * (math.ceil(tokens / rows / page_size) + 1),
                len(ones) + sum(math.ceil(n / page_size) for n in portion))
    cache = CacheManager(entries, page_size, max_seqs, max_model_len, dtype, device, pages=pages)
    runner, sampler = Runner(model, cache, ctx, max_step_tokens), Sampler(ctx.kernels, device)
    params = SamplingParams(temperature=1.0)

    def step(counts) -> None:
        batch = []
        for n in counts:
            slot = cache.admit()
            cache.reserve(slot, n)
            batch.append(StepEntry(slot, [0] * n, 0, (n - 1,)))
        arrays = sampling_arrays([(params, 1, n) for n in counts])
        arrays["sample_slot"] = np.array([e.slot for e in batch], dtype=np.int32)
        ctx_ = runner.context(batch, extra=arrays)
        logits = model.forward(ctx_)
        sampler.sample(logits, ctx_.extra, False)
        for e in batch:
            cache.release(e.slot)

    share = [tokens // rows + (i < tokens % rows) for i in range(rows)]
    largest = _peak_of(device, lambda: step([n for n in share if n]))
    graphed = _peak_of(device, lambda: step(ones + [n for n in portion if n > 0]))
    del runner, cache
    torch.cuda.empty_cache()
    return largest, graphed


def build(source, *, dtype: str, device, kernels=None, page_size: int, max_seqs: int, max_model_len: int,
          max_step_tokens: int, state_memory: int | None = None, pages: int | None = None,
          memory_fraction: float = 0.9, prefix_cache: bool = False, chunk_with_decode: int = 0,
          cuda_graphs: bool = True) -> Built:
    """`kernels=None` loads the compiled CUDA kernels and fails if they cannot be had. With neither `state_memory`
    nor `pages` the cache pools take `memory_fraction` of the device memory that is free after the weights, less the
    measured activation peak of the largest step and (with `cuda_graphs`) of the largest step that graphs replay,
    whose pool stays reserved."""
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
    activations = graphs = free_before = None
    if state_memory is None and pages is None:
        if device.type != "cuda":
            raise ValueError("only a CUDA device's free memory can be measured: give state_memory or pages")
        with torch.inference_mode():
            activations, graphs = _measure(model, ctx, model.entries, page_size=page_size, max_seqs=max_seqs,
                                           max_model_len=max_model_len, max_step_tokens=max_step_tokens,
                                           chunk_with_decode=chunk_with_decode, dtype=tdtype, device=device)
        if not cuda_graphs:
            graphs = 0
        free_before, _ = torch.cuda.mem_get_info(device)
        state_memory = int(free_before * memory_fraction) - activations - graphs
    cache = CacheManager(model.entries, page_size, max_seqs, max_model_len, tdtype, device,
                         state_memory=state_memory, pages=pages, prefix_cache=prefix_cache)
    free_after = torch.cuda.mem_get_info(device)[0] if device.type == "cuda" else None
    memory = Memory(weight_bytes, cache.bytes, activations, graphs, free_before, free_after)
    return Built(config, model, cache, Runner(model, cache, ctx, max_step_tokens), ctx, weight_bytes, memory)
