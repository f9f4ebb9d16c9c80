"""One registry from an architecture's name (config.json's `architectures[0]`) to its
configuration class. The configuration class yields the `ModelSpec`; the generic
model runtime builds itself from that, so registering a configuration class is all
that adding an architecture takes.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Mapping

_ARCHITECTURES: dict[str, type] = {}
_MODEL_TYPES: dict[str, str] = {}


class ModelConfig:
    """Base of every architecture's typed configuration.

    A subclass is a frozen dataclass whose fields are the architecture's own
    config.json keys. It provides:
      from_dict(mapping)  typed reads, defaults, validation errors that name the key
      to_dict()           the config.json to write beside random weights
      model_spec()        the architecture-neutral `ModelSpec`
    """
    architecture: str = ""
    model_type: str = ""

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> dict:
        raise NotImplementedError

    def model_spec(self):
        raise NotImplementedError


def register_architecture(name: str, config_class: type, model_type: str | None = None) -> None:
    """Register `config_class` under config.json's architecture name (and, for files
    without an `architectures` key, under its `model_type`)."""
    if name in _ARCHITECTURES and _ARCHITECTURES[name] is not config_class:
        raise ValueError(f"architecture {name!r} is already registered to {_ARCHITECTURES[name].__name__}")
    _ARCHITECTURES[name] = config_class
    if model_type:
        _MODEL_TYPES[model_type] = name


def registered_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def config_class_for(data: Mapping[str, Any]) -> type:
    names = data.get("architectures") or []
    if isinstance(names, str):
        names = [names]
    name = names[0] if names else _MODEL_TYPES.get(str(data.get("model_type", "")))
    if name not in _ARCHITECTURES:
        raise ValueError(
            f"unknown architecture {name!r} (model_type {data.get('model_type')!r}); "
            f"registered: {', '.join(registered_architectures()) or 'none'}")
    return _ARCHITECTURES[name]


def config_from_dict(data: Mapping[str, Any]) -> ModelConfig:
    return config_class_for(data).from_dict(data)


def load_config(model_dir) -> ModelConfig:
    """Read `<model_dir>/config.json` and build the registered configuration for it."""
    path = Path(model_dir) / "config.json"
    if not path.exists():
        raise FileNotFoundError(f"config.json not found in {model_dir}")
    return config_from_dict(json.loads(path.read_text(encoding="utf-8")))
