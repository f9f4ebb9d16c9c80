"""RMSNorm: x * rsqrt(mean(x^2) + eps) * w, statistics in float32 (student_engine.py:530-535).

The residual stream is float32 in both precisions; the addition of the previous part's output
is fused into this kernel, so the stream is read once and written once per norm."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import Norm, TensorSpec
from .registry import register_part


class RmsNorm(Norm):
    """params: width, eps. tensors: weight [width]."""

    def __init__(self, spec):
        super().__init__(spec)
        self.width = int(self.params["width"])
        self.eps = float(self.params["eps"])
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.file_name("weight"), (self.width,), init="norm")]

    def kernel_libraries(self, dtype):
        return {"norm"}

    def bind(self, tensors, dtype, device):
        self.weight = tensors[self.file_name("weight")]

    def forward(self, hidden: torch.Tensor, delta: Optional[torch.Tensor]) -> torch.Tensor:
        out = torch.empty(hidden.shape, dtype=self.weight.dtype, device=hidden.device)
        ops.add_rms_norm(hidden, delta, self.weight, self.eps, out)
        return out

    def fused_rms(self):
        return self.weight, self.eps

    def step_weights(self):
        return [self.weight]


register_part("norm", "rms_norm", RmsNorm)
