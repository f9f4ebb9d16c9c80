"""Random-weights mode: from a configuration and a seed to a model folder (config.json and
model.safetensors) that loads like any other.

Every tensor is drawn in float32 on the CPU from one seeded generator, in the order in which the
model's parts name them, then stored in `store_dtype`: matrices, tables and biases N(0, 0.02), norm
weights 1 + N(0, 0.1). The draws do not depend on the device or on the compute precision."""
from __future__ import annotations

import json
from pathlib import Path

import torch

from ..config.registry import ModelConfig
from ..parts.base import TensorSpec
from .loader import merge_specs
from .safetensors_io import save_safetensors


def draw_tensor(spec: TensorSpec, generator: torch.Generator, store_dtype: torch.dtype) -> torch.Tensor:
    if spec.keep == "int32":
        return torch.zeros(spec.shape, dtype=torch.int32)
    noise = torch.randn(spec.shape, generator=generator, dtype=torch.float32)
    if spec.init == "norm":
        value = 1.0 + 0.1 * noise
    elif spec.init in ("matrix", "bias"):
        value = 0.02 * noise
    else:
        raise ValueError(f"tensor {spec.name!r}: unknown init {spec.init!r}")
    return value if spec.keep == "stored" else value.to(store_dtype)


def random_state(specs, seed: int, store_dtype: torch.dtype = torch.bfloat16) -> dict[str, torch.Tensor]:
    generator = torch.Generator().manual_seed(int(seed))
    return {name: draw_tensor(spec, generator, store_dtype) for name, spec in merge_specs(specs).items()}


def random_state_on_device(specs, seed: int, dtype: torch.dtype, device) -> dict[str, torch.Tensor]:
    """The same distributions drawn on `device` by its own generator, tensor by tensor, straight into the kept
    dtype: for measurements at sizes whose model file would take minutes to write and read (tens of GB). The values
    are NOT those of `random_state` with the same seed; nothing that is compared with a model folder uses this."""
    generator = torch.Generator(device=device).manual_seed(int(seed))
    out = {}
    for name, spec in merge_specs(specs).items():
        if spec.keep == "int32":
            out[name] = torch.zeros(spec.shape, dtype=torch.int32, device=device)
            continue
        if spec.init not in ("norm", "matrix", "bias"):
            raise ValueError(f"tensor {spec.name!r}: unknown init {spec.init!r}")
        kept = torch.float32 if spec.keep == "stored" else dtype
        value = torch.empty(spec.shape, dtype=kept, device=device)
        flat = value.view(-1)
        for begin in range(0, flat.numel(), 1 << 27):  # float32 draws of at most 512 MB at a time
            noise = torch.randn(min(1 << 27, flat.numel() - begin), generator=generator, dtype=torch.float32, device=device)
            noise = 1.0 + 0.1 * noise if spec.init == "norm" else 0.02 * noise
            flat[begin:begin + noise.numel()] = noise.to(kept)
        out[name] = value
    return out


def write_random_model(config: ModelConfig, seed: int, out_dir, store_dtype: torch.dtype = torch.bfloat16) -> Path:
    """Write `<out_dir>/config.json` and `<out_dir>/model.safetensors`; returns out_dir."""
    from ..engine.model import Model  # late import: the model needs the weights package

    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    specs = Model.tensor_specs_of(config.model_spec())
    data = config.to_dict()
    data["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32"}.get(store_dtype, str(store_dtype))
    (out_dir / "config.json").write_text(json.dumps(data, indent=1), encoding="utf-8")
    save_safetensors(out_dir / "model.safetensors", random_state(specs, seed, store_dtype))
    return out_dir
