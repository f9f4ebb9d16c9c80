"""Where a model lives: a local folder, or the newest snapshot of a hub id in the local hub cache
(`$HF_HUB_CACHE`, `$HF_HOME/hub`, `~/.cache/huggingface/hub`), as the reference resolves it
(utils/load_weights.py:12-38). Nothing is ever downloaded."""
from __future__ import annotations

import os
from pathlib import Path


def resolve_model_dir(model_path) -> Path:
    candidate = Path(model_path)
    if candidate.exists():
        return candidate
    text = str(model_path)
    if "/" not in text:
        raise FileNotFoundError(f"Model path not found: {model_path}")
    if os.environ.get("HF_HUB_CACHE"):
        root = Path(os.environ["HF_HUB_CACHE"])
    elif os.environ.get("HF_HOME"):
        root = Path(os.environ["HF_HOME"]) / "hub"
    else:
        root = Path(os.path.expanduser("~")) / ".cache" / "huggingface" / "hub"
    namespace, name = text.split("/", 1)
    snapshots = root / f"models--{namespace}--{name}" / "snapshots"
    if not snapshots.exists():
        raise FileNotFoundError(f"Model cache not found: {snapshots.parent}")
    found = sorted(p for p in snapshots.iterdir() if p.is_dir())
    if not found:
        raise FileNotFoundError(f"No snapshots found under {snapshots}")
    return found[-1]
