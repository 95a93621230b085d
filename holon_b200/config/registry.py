"""One registry from an architecture's name (`config.json`: `architectures[0]`) to its typed configuration and recipe.

The reference resolves `arch.<name>` to exactly one model plugin and refuses duplicates
(core/holon/core/plugins.py:31-66, 207-212); this registry keeps both rules in one process.
"""
from __future__ import annotations

import dataclasses
from collections.abc import Callable, Mapping
from typing import Any

from .spec import ModelSpec


class ConfigError(ValueError):
    """config.json lacks a key, holds a value of the wrong kind, or asks for what the architecture does not have."""


@dataclasses.dataclass(frozen=True)
class Architecture:
    name: str
    parse: Callable[[Mapping[str, Any]], Any]            # config.json dict -> typed configuration
    recipe: Callable[[Any], ModelSpec]                    # typed configuration -> ModelSpec


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, parse, recipe, replace: bool = False) -> Architecture:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is registered already")
    _ARCHITECTURES[name] = arch = Architecture(name, parse, recipe)
    return arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def architectures() -> tuple[str, ...]:
    return tuple(sorted(_ARCHITECTURES))


def resolve_architecture(config: Mapping[str, Any]) -> Architecture:
    """The architecture `config.json` names. Importing `holon_b200.models` registers the built-in ones."""
    from .. import models  # noqa: F401  (registration on import)
    names = config.get("architectures")
    if not isinstance(names, (list, tuple)) or not names:
        raise ConfigError("config.json: 'architectures' must be a list with the model class's name first")
    if names[0] not in _ARCHITECTURES:
        raise ConfigError(f"config.json: architecture {names[0]!r} is not registered; known: {list(architectures())}")
    return _ARCHITECTURES[names[0]]
