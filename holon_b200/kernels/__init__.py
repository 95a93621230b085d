"""The kernels of the product path. `load_kernels(device)` compiles them on first use and fails loudly when that
cannot be done or the device is no CUDA device; nothing falls back to another implementation."""
from __future__ import annotations

from .build import BuildError, library_path

_LOADED: dict = {}


def load_kernels(device):
    import torch
    from .cuda import CudaKernels, KernelError
    device = torch.device(device)
    if device.type != "cuda":
        raise KernelError(f"holon_b200 runs on CUDA devices only; asked for {device}")
    if not torch.cuda.is_available():
        raise KernelError("holon_b200 needs a CUDA device and found none (torch.cuda.is_available() is False)")
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    if device not in _LOADED:
        _LOADED[device] = CudaKernels(device)
    return _LOADED[device]


__all__ = ["BuildError", "library_path", "load_kernels"]
