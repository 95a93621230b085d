"""Layers put together from parts: mixers, feed-forwards, norms, position encodings, blocks, and the model that
arranges them by a run order."""
from . import _builtin  # noqa: F401
from .base import BuildContext, PagedKV, Param, Part, Residual, SlotState, register_part, unregister_part
from .model import CacheEntry, LayerCache, Model

__all__ = ["BuildContext", "CacheEntry", "LayerCache", "Model", "PagedKV", "Param", "Part", "Residual", "SlotState",
           "register_part", "unregister_part"]
