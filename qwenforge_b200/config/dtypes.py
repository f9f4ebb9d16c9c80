"""Names of the compute precisions, in the reference's spelling
(student_engine.py:480-496: auto, float16/fp16/half, bfloat16/bf16, float32/fp32).

This library keeps weights in bfloat16 or runs everything in true float32; float16 is
recognised and refused with a message that says so.
"""
from __future__ import annotations

import torch

_NAMES = {
    "float16": torch.float16, "fp16": torch.float16, "half": torch.float16,
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float32": torch.float32, "fp32": torch.float32,
}


def resolve_dtype(dtype, config_torch_dtype: str | None = None) -> torch.dtype:
    """'auto' takes config.json's torch_dtype (float16 there falls to bfloat16: the same
    16-bit weight footprint in the format this library keeps); anything else is looked
    up by name."""
    if isinstance(dtype, torch.dtype):
        resolved = dtype
    else:
        name = str(dtype).lower()
        if name == "auto":
            name = str(config_torch_dtype or "bfloat16").lower()
            if name in ("float16", "fp16", "half"):
                name = "bfloat16"
        if name not in _NAMES:
            raise ValueError(f"Unsupported dtype: {dtype}")
        resolved = _NAMES[name]
    if resolved == torch.float16:
        raise ValueError("Unsupported dtype: float16 (this library computes in bfloat16 or float32; "
                         "pass --dtype bfloat16 for the fast path or float32 for the exact one)")
    if resolved not in (torch.bfloat16, torch.float32):
        raise ValueError(f"Unsupported dtype: {dtype}")
    return resolved
