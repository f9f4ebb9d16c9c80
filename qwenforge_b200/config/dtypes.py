"""Names of the compute precisions, in the reference's spelling
(student_engine.py:480-496: auto, float16/fp16/half, bfloat16/bf16, float32/fp32).

This library keeps weights in bfloat16 or runs everything in true float32. The reference's default is float16;
its users pass that name, so the name is accepted and served by the 16-bit path this library has, bfloat16
(the same footprint and tensor-core rate, a wider exponent), with one warning that says so.
"""
from __future__ import annotations

import warnings

import torch

_NAMES = {
    "float16": torch.float16, "fp16": torch.float16, "half": torch.float16,
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float32": torch.float32, "fp32": torch.float32,
}


def resolve_dtype(dtype, config_torch_dtype: str | None = None) -> torch.dtype:
    """'auto' takes config.json's torch_dtype; anything else is looked up by name. float16 resolves to bfloat16."""
    asked_for_half = False
    if isinstance(dtype, torch.dtype):
        resolved = dtype
    else:
        name = str(dtype).lower()
        if name == "auto":
            name = str(config_torch_dtype or "bfloat16").lower()
        else:
            asked_for_half = name in ("float16", "fp16", "half")
        if name not in _NAMES:
            raise ValueError(f"Unsupported dtype: {dtype}")
        resolved = _NAMES[name]
    if resolved == torch.float16:
        if asked_for_half or isinstance(dtype, torch.dtype):
            warnings.warn("float16 was asked for: this library's 16-bit path is bfloat16, which is used instead "
                          "(pass float32 for the exact path)", stacklevel=2)
        resolved = torch.bfloat16
    if resolved not in (torch.bfloat16, torch.float32):
        raise ValueError(f"Unsupported dtype: {dtype}")
    return resolved
