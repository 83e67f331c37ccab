"""Typed model configuration read from a checkpoint's ``config.json``.

A configuration class declares its fields as dataclass fields.  Every field is
read from the JSON key of the same name; a field without a default is required.
Nothing about a model's sizes lives in code: kernels, parts and the cache get
their sizes from an instance of one of these classes.

The reference pins its sizes in a compiled registry and checks GGUF metadata
against it (src/kipp.c:756-795, src/kipp_checkpoints.h:25-79); here the
checkpoint's own ``config.json`` is the single source.
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Any, ClassVar


class ConfigError(ValueError):
    """A ``config.json`` is missing a key, has a wrong type, or asks for an
    option the engine does not implement."""


_MISSING = dataclasses.MISSING


def _coerce(name: str, value: Any, annotation: Any) -> Any:
    """Check ``value`` against the annotation of a field (a string under
    ``from __future__ import annotations``, else the type itself)."""
    if not isinstance(annotation, str):
        annotation = getattr(annotation, "__name__", None) or str(annotation).replace("typing.", "")
    base = annotation.replace("Optional[", "").replace("]", "").strip()
    optional = annotation.startswith("Optional[") or "| None" in annotation
    base = base.replace("| None", "").strip()
    if value is None:
        if optional:
            return None
        raise ConfigError(f"config key {name!r} must not be null")
    if base == "int":
        if isinstance(value, bool) or not isinstance(value, int):
            if isinstance(value, float) and float(value).is_integer():
                return int(value)
            raise ConfigError(f"config key {name!r} must be an integer, got {value!r}")
        return int(value)
    if base == "float":
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"config key {name!r} must be a number, got {value!r}")
        return float(value)
    if base == "bool":
        if not isinstance(value, bool):
            raise ConfigError(f"config key {name!r} must be true or false, got {value!r}")
        return value
    if base == "str":
        if not isinstance(value, str):
            raise ConfigError(f"config key {name!r} must be a string, got {value!r}")
        return value
    if base.startswith("tuple"):
        if not isinstance(value, (list, tuple)):
            raise ConfigError(f"config key {name!r} must be a list, got {value!r}")
        return tuple(value)
    return value


@dataclasses.dataclass(frozen=True)
class ModelConfig:
    """Base of all architecture configurations.

    Subclasses add fields and override :meth:`validate`.  ``architecture`` is
    the value of ``architectures[0]`` in ``config.json`` and selects the model
    class through :mod:`kipp_b200.config.registry`.
    """

    architecture: str

    # JSON keys that are read under another name.
    json_aliases: ClassVar[dict[str, tuple[str, ...]]] = {}

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "ModelConfig":
        if not isinstance(data, dict):
            raise ConfigError("config.json must hold a JSON object")
        archs = data.get("architectures")
        if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
            raise ConfigError("config.json lacks 'architectures': [name]")
        values: dict[str, Any] = {"architecture": archs[0]}
        for field in dataclasses.fields(cls):
            if field.name == "architecture":
                continue
            keys = (field.name,) + tuple(cls.json_aliases.get(field.name, ()))
            present = [k for k in keys if k in data]
            if present:
                values[field.name] = _coerce(present[0], data[present[0]], field.type)
            elif field.default is _MISSING and field.default_factory is _MISSING:
                raise ConfigError(f"config.json lacks required key {field.name!r}")
        config = cls(**values)
        config.validate()
        return config

    def validate(self) -> None:  # pragma: no cover - overridden
        pass

    def to_dict(self) -> dict[str, Any]:
        """The JSON form that :meth:`from_dict` reads back to an equal object."""
        out: dict[str, Any] = {"architectures": [self.architecture]}
        for field in dataclasses.fields(self):
            if field.name == "architecture":
                continue
            value = getattr(self, field.name)
            out[field.name] = list(value) if isinstance(value, tuple) else value
        return out

    def save(self, folder: str) -> None:
        os.makedirs(folder, exist_ok=True)
        with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
            json.dump(self.to_dict(), f, indent=2)
            f.write("\n")


def read_config_json(folder: str) -> dict[str, Any]:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{folder}: no config.json")
    with open(path, "r", encoding="utf-8") as f:
        try:
            return json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
