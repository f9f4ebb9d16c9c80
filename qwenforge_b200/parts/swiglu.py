"""SwiGLU feed-forward: (silu(x Wg^T) * (x Wu^T)) Wd^T, no biases (student_engine.py:523-527, :663-666).
Gate and up weights are concatenated by rows so that one product yields both halves."""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, TensorSpec
from .registry import register_part


class SwiGlu(FeedForward):
    """params: hidden_size, intermediate_size. tensors: gate_weight [I, W], up_weight [I, W], down_weight [W, I]."""

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.params["hidden_size"])
        self.inter = int(self.params["intermediate_size"])
        self.gate_up_weight = self.down_weight = None

    def tensor_specs(self):
        return [
            TensorSpec(self.file_name("gate_weight"), (self.inter, self.hidden)),
            TensorSpec(self.file_name("up_weight"), (self.inter, self.hidden)),
            TensorSpec(self.file_name("down_weight"), (self.hidden, self.inter)),
        ]

    def kernel_libraries(self, dtype):
        return {"activation"} | ({"gemm_f32"} if dtype == torch.float32 else set())

    def bind(self, tensors, dtype, device):
        self.gate_up_weight = torch.cat((tensors[self.file_name("gate_weight")], tensors[self.file_name("up_weight")]),
                                        dim=0).contiguous()
        self.down_weight = tensors[self.file_name("down_weight")]

    def forward(self, x, ctx):
        gate_up = ops.linear(x, self.gate_up_weight)
        act = torch.empty((x.shape[0], self.inter), dtype=x.dtype, device=x.device)
        ops.swiglu(gate_up, act)
        return ops.linear(act, self.down_weight)


register_part("feed_forward", "swiglu", SwiGlu)
