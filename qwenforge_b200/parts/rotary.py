"""Split-half rotary position encoding (student_engine.py:362-363, :537-554).

inv_freq_j = theta^(-2j/R), j < R/2, formed in float32 on the host exactly as the reference
forms it; the angle float32(position) * inv_freq_j and its sine and cosine are float32 in the
kernel. Component j pairs with component j + R/2 (`rotate_half`). R (`rotary_dim`) defaults
to the head size."""
from __future__ import annotations

import torch

from .base import PositionEncoding
from .registry import register_part


class RotaryHalf(PositionEncoding):
    """params: head_dim, theta, rotary_dim (optional). No tensors in the weight files."""

    def __init__(self, spec):
        super().__init__(spec)
        self.head_dim = int(self.params["head_dim"])
        self.rotary_dim = int(self.params.get("rotary_dim") or self.head_dim)
        self.theta = float(self.params["theta"])
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary_half: rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        self.inv_freq = None

    def bind(self, tensors, dtype, device):
        index = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32)
        self.inv_freq = (1.0 / (self.theta ** (index / self.rotary_dim))).to(device)

    def fused_rotary(self):
        return self.inv_freq, self.rotary_dim


register_part("position", "rotary_half", RotaryHalf)
