"""One registry from an architecture name to its configuration class and its
model builder.

``architectures[0]`` of ``config.json`` is the key.  The reference knows a
single architecture string and refuses everything else with an "unsupported"
error (src/kipp.c:756-760); this registry does the same for unknown names and
is where another architecture is added: ``register_architecture(name, config
class, builder)`` with ``builder(config) -> ModelSpec``.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Callable, Type

from .base import ConfigError, ModelConfig, read_config_json


@dataclasses.dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Type[ModelConfig]
    build: Callable[[ModelConfig], Any]   # -> kipp_b200.models.spec.ModelSpec


_REGISTRY: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: Type[ModelConfig],
                          build: Callable[[ModelConfig], Any], *, replace: bool = False) -> None:
    if name in _REGISTRY and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    _REGISTRY[name] = Architecture(name, config_class, build)


def unregister_architecture(name: str) -> None:
    _REGISTRY.pop(name, None)


def registered_architectures() -> list[str]:
    _ensure_builtin()
    return sorted(_REGISTRY)


def is_registered(name: str) -> bool:
    _ensure_builtin()
    return name in _REGISTRY


def get_architecture(name: str) -> Architecture:
    _ensure_builtin()
    try:
        return _REGISTRY[name]
    except KeyError:
        raise ConfigError(
            f"unsupported architecture {name!r}; registered: {sorted(_REGISTRY)}") from None


def config_from_dict(data: dict) -> ModelConfig:
    archs = data.get("architectures") if isinstance(data, dict) else None
    if not isinstance(archs, list) or not archs:
        raise ConfigError("config.json lacks 'architectures': [name]")
    return get_architecture(archs[0]).config_class.from_dict(data)


def load_config(folder: str) -> ModelConfig:
    """Read ``folder/config.json`` into the typed configuration of its architecture."""
    return config_from_dict(read_config_json(folder))


_builtin_done = False


def _ensure_builtin() -> None:
    global _builtin_done
    if _builtin_done:
        return
    _builtin_done = True
    from ..models import qwen3  # noqa: F401  (registers itself on import)
