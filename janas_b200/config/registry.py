"""One registry from an architecture's name to its configuration class.

``config.json`` names the architecture (``architectures[0]``, else
``model_type``); the class found here reads the file's keys and turns them into
a ``ModelSpec`` from which the one generic decoder is built.  The reference
looks the name up in a static table in the same way and fails with
"architecture ... not supported" (src/llm/arch.c:10-66,
src/llm/model_load.c:800-804).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Mapping, Protocol

from .spec import ConfigError, ModelSpec


class ArchitectureConfig(Protocol):
    """What a configuration class must offer to be registered."""

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "ArchitectureConfig": ...

    def to_dict(self) -> Dict[str, Any]: ...

    def to_model_spec(self) -> ModelSpec: ...


_ARCHITECTURES: Dict[str, type] = {}
_MODEL_TYPES: Dict[str, str] = {}


def register_architecture(name: str, config_cls: type, model_type: str | None = None) -> None:
    """Make ``name`` (as ``config.json`` spells it) known; ``model_type`` is
    the fallback key for folders that give no ``architectures`` list."""
    _ARCHITECTURES[name] = config_cls
    if model_type is not None:
        _MODEL_TYPES[model_type] = name


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def architecture_name(d: Mapping[str, Any]) -> str:
    archs = d.get("architectures")
    if archs:
        return str(archs[0])
    mt = d.get("model_type")
    if mt in _MODEL_TYPES:
        return _MODEL_TYPES[mt]
    raise ConfigError("config.json names no architecture (architectures, model_type)")


def config_from_dict(d: Mapping[str, Any]):
    name = architecture_name(d)
    cls = _ARCHITECTURES.get(name)
    if cls is None:
        raise ConfigError(f"architecture {name!r} is not supported; known: "
                          + ", ".join(known_architectures()))
    return cls.from_dict(d)


def config_from_dir(model_dir: str):
    """The typed configuration of the model folder ``model_dir``."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir}: no config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: not a JSON object")
    return config_from_dict(d)
