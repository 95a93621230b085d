"""Typed configuration: the model description a recipe returns, the architecture registry, the engine settings."""
from .engine import EngineConfig
from .registry import (Architecture, ConfigError, architectures, register_architecture, resolve_architecture,
                       unregister_architecture)
from .spec import LayerSpec, ModelSpec, PartRef, Run, WeightRule

__all__ = ["Architecture", "ConfigError", "EngineConfig", "LayerSpec", "ModelSpec", "PartRef", "Run", "WeightRule",
           "architectures", "register_architecture", "resolve_architecture", "unregister_architecture"]
