"""Named configurations kept as config.json files beside this module (data, not code):
the two tiny test sizes and the Qwen2.5 0.5B / 3B / 7B layer sizes. They serve the
random-weights mode, the tests and the measurement, where no model folder exists."""
from __future__ import annotations

import json
from pathlib import Path

from .registry import ModelConfig, config_from_dict

_DIR = Path(__file__).parent / "presets"


def preset_names() -> list[str]:
    return sorted(p.stem for p in _DIR.glob("*.json"))


def preset_dict(name: str) -> dict:
    path = _DIR / f"{name.lower()}.json"
    if not path.exists():
        raise ValueError(f"unknown preset {name!r}; available: {', '.join(preset_names())}")
    return json.loads(path.read_text(encoding="utf-8"))


def preset_config(name: str, **overrides) -> ModelConfig:
    data = preset_dict(name)
    data.update(overrides)
    return config_from_dict(data)
