"""Weights by tensor name.

`load_weights(model_dir, specs, dtype, device)` reads the tensors that the model's parts ask for
(`TensorSpec`s) from the folder's safetensors files and keeps each in its kept dtype:
  keep="compute"  the activation dtype: bfloat16, or float32 on the 32-bit path
  keep="stored"   as the file stores it when that is a 32-bit float, else like "compute"
  keep="int32"    integer tables as int32
Anything that does not line up is reported in ONE `WeightsError` that lists every missing
tensor, every unexpected tensor and every wrong shape. The file layout follows the reference's
loader (utils/load_weights.py:49-73): `model.safetensors.index.json`'s `weight_map` if present,
else every `*.safetensors` in the folder, and a name found in two files is an error.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Iterable, Mapping, Optional, Sequence

import torch

from ..parts.base import TensorSpec
from .safetensors_io import SafetensorsFile


class WeightsError(ValueError):
    def __init__(self, message: str, missing=(), unexpected=(), wrong_shape=(), wrong_dtype=(), duplicated=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        self.duplicated = list(duplicated)


def weight_files(model_dir) -> list[Path]:
    model_dir = Path(model_dir)
    if not model_dir.is_dir():
        raise FileNotFoundError(f"Model path not found: {model_dir}")
    index = model_dir / "model.safetensors.index.json"
    if index.exists():
        names = sorted(set(json.loads(index.read_text(encoding="utf-8")).get("weight_map", {}).values()))
        files = [model_dir / n for n in names]
        absent = [str(f) for f in files if not f.exists()]
        if absent:
            raise FileNotFoundError(f"weight files named by the index are missing: {', '.join(absent)}")
        return files
    files = sorted(model_dir.glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"No safetensors files found in {model_dir}")
    return files


def merge_specs(specs: Iterable[TensorSpec]) -> dict[str, TensorSpec]:
    """One spec per file name; two parts may name the same tensor (tied tables) if they agree on it."""
    merged: dict[str, TensorSpec] = {}
    for spec in specs:
        seen = merged.get(spec.name)
        if seen is None:
            merged[spec.name] = spec
        elif tuple(seen.shape) != tuple(spec.shape) or seen.keep != spec.keep:
            raise ValueError(f"tensor {spec.name!r} is wanted as {tuple(seen.shape)}/{seen.keep} "
                             f"and as {tuple(spec.shape)}/{spec.keep}")
    return merged


def kept_dtype(spec: TensorSpec, stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    if spec.keep == "int32":
        return torch.int32
    if spec.keep == "stored" and stored == torch.float32:
        return torch.float32
    return compute


def _list(items: Sequence[str], limit: int = 12) -> str:
    items = list(items)
    shown = ", ".join(items[:limit])
    return shown + (f", ... ({len(items) - limit} more)" if len(items) > limit else "")


def load_weights(model_dir, specs: Iterable[TensorSpec], dtype: torch.dtype, device,
                 redundant: Optional[Mapping[str, str]] = None) -> dict[str, torch.Tensor]:
    """`redundant`: names the files may hold beyond the wanted ones, each mapped to the wanted tensor it must equal."""
    wanted = merge_specs(specs)
    redundant = dict(redundant or {})
    files = [SafetensorsFile(p) for p in weight_files(model_dir)]
    try:
        where: dict[str, SafetensorsFile] = {}
        duplicated = []
        for f in files:
            for name in f.names():
                if name in where:
                    duplicated.append(name)
                where[name] = f
        source = {n: (n if n in where or s.fallback not in where else s.fallback) for n, s in wanted.items()}
        missing = sorted(n for n in wanted if source[n] not in where)
        unexpected = sorted(n for n in where if n not in wanted and n not in redundant)
        wrong_shape, wrong_dtype = [], []
        for extra, twin in redundant.items():
            if extra in where and extra not in wanted and twin in where:
                if where[extra].info(extra)[1] != where[twin].info(twin)[1] or not torch.equal(
                        where[extra].tensor(extra), where[twin].tensor(twin)):
                    wrong_shape.append(f"{extra}: the files hold it although the model shares {twin}, and it differs from that")
        for name, spec in wanted.items():
            if source[name] not in where:
                continue
            name = source[name]
            stored_dtype, shape = where[name].info(name)
            if tuple(shape) != tuple(spec.shape):
                wrong_shape.append(f"{name}: file has {list(shape)}, model wants {list(spec.shape)}")
            is_int = not stored_dtype.is_floating_point
            if is_int != (spec.keep == "int32"):
                wrong_dtype.append(f"{name}: file stores {stored_dtype}, model wants "
                                   f"{'an integer table' if spec.keep == 'int32' else 'a floating-point tensor'}")
        if missing or unexpected or wrong_shape or wrong_dtype or duplicated:
            lines = [f"weights in {model_dir} do not match the model:"]
            if missing:
                lines.append(f"  missing ({len(missing)}): {_list(missing)}")
            if unexpected:
                lines.append(f"  unexpected ({len(unexpected)}): {_list(unexpected)}")
            if wrong_shape:
                lines.append(f"  wrong shape ({len(wrong_shape)}): {_list(wrong_shape)}")
            if wrong_dtype:
                lines.append(f"  wrong dtype ({len(wrong_dtype)}): {_list(wrong_dtype)}")
            if duplicated:
                lines.append(f"  in more than one file ({len(duplicated)}): {_list(sorted(duplicated))}")
            raise WeightsError("\n".join(lines), missing, unexpected, wrong_shape, wrong_dtype, duplicated)
        out = {}
        for name, spec in wanted.items():
            held = source[name]
            if held != name and held in out:
                out[name] = out[held]      # the stand-in is wanted under its own name too: one tensor on the device
                continue
            stored_dtype, _ = where[held].info(held)
            out[name] = where[held].tensor(held).to(device=device, dtype=kept_dtype(spec, stored_dtype, dtype))
        return out
    finally:
        for f in files:
            f.close()
