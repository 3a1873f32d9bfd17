"""One table from an architecture's name to its configuration class and model recipe.

``config.json``'s ``architectures[0]`` (or, when absent, ``model_type``) chooses the
entry; every entry point of the engine resolves a model folder through here, as the
reference resolves ``model_type`` to an adapter (python/instinct/backends/factory.py:12-27).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

from .model_config import ConfigError, ModelConfig


@dataclass(frozen=True)
class Architecture:
    name: str
    config_from_json: Callable[[dict[str, Any]], ModelConfig]
    # (config) -> parts.model.ModelRecipe; imported lazily by the caller.
    recipe: Callable[[ModelConfig], Any]
    model_types: tuple[str, ...] = ()


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(
    name: str,
    config_from_json: Callable[[dict[str, Any]], ModelConfig],
    recipe: Callable[[ModelConfig], Any],
    *,
    model_types: tuple[str, ...] = (),
    replace: bool = False,
) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture '{name}' is already registered")
    _ARCHITECTURES[name] = Architecture(name, config_from_json, recipe, tuple(model_types))


def registered_architectures() -> tuple[str, ...]:
    return tuple(sorted(_ARCHITECTURES))


def resolve_architecture(raw_config: dict[str, Any]) -> Architecture:
    names = raw_config.get("architectures") or []
    if names:
        name = names[0]
        if name not in _ARCHITECTURES:
            raise ConfigError(
                f"no model registered for '{name}' (registered: "
                f"{', '.join(registered_architectures()) or 'none'})"
            )
        return _ARCHITECTURES[name]
    model_type = raw_config.get("model_type")
    for entry in _ARCHITECTURES.values():
        if model_type in entry.model_types:
            return entry
    raise ConfigError(
        f"config.json names no architecture and model_type {model_type!r} is not registered"
    )


def parse_config(raw_config: dict[str, Any]) -> tuple[Architecture, ModelConfig]:
    entry = resolve_architecture(raw_config)
    return entry, entry.config_from_json(raw_config)
