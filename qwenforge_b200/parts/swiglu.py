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
        return {"activation"} | ({"gemm_f32"} if dtype == torch.float32 else {"skinny_gemm", "tc_gemm", "wide_gemm"})

    def bind(self, tensors, dtype, device):
        self.gate_up_weight = torch.cat((tensors[self.file_name("gate_weight")], tensors[self.file_name("up_weight")]),
                                        dim=0).contiguous()
        self.down_weight = tensors[self.file_name("down_weight")]

    def step_weights(self):
        return [self.gate_up_weight, self.down_weight]

    def forward(self, x, ctx):
        act = torch.empty((x.shape[0], self.inter), dtype=x.dtype, device=x.device)
        # Steps with tiles for every SM run gate/up with the gate in the product's epilogue on this library's
        # persistent tcgen05 kernel: measured at 2048 x 9728 x 896 it takes 36 microseconds where the library product
        # (31) and the gate kernel after it take 46, since the product's 40 MB of output are never written and read.
        own = x.dtype == torch.bfloat16 and self.inter % 8 == 0 and ops.tc_gemm_takes(x, self.gate_up_weight) and (
            ops.own_tensor_core_products(x, self.gate_up_weight)
            or ops.tc_gemm_is_persistent(ops.TC_SWIGLU, x.shape[0], 2 * self.inter))
        if own:
            ops.tc_gemm(ops.TC_SWIGLU, x, self.gate_up_weight, act, ctx.err if ctx is not None else None)
            return ops.linear(act, self.down_weight)
        gate_up = ops.linear(x, self.gate_up_weight)
        ops.swiglu(gate_up, act)
        return ops.linear(act, self.down_weight)

    # ---- the form for steps of up to 64 tokens that works on the residual stream in place: norm + gate/up + SwiGLU in
    # one kernel, down + residual in another. Each of the two products goes the way that is fastest by measurement
    # (`python -m qwenforge_b200.measure products`). Gate/up: the mma.sync streamer where it takes the shape and pays
    # (`ops.skinny_gemm_pays`); the tcgen05 streamer after the norm kernel for weights of 100 MB and more (Qwen2.5-7B:
    # 50 microseconds against 52 unfused and 56 to 62 in the mma.sync streamer); else norm kernel, library product and
    # gate kernel. Down: `ops.residual_product_way`.
    def _ways(self, ctx):
        rows = ctx.n_tokens
        gate_up = "unfused"
        if (rows <= ops.SKINNY_MAX_ROWS and ops.skinny_gemm_takes(rows, self.gate_up_weight, ops.EPI_SWIGLU, True)
                and ops.skinny_gemm_pays(rows, self.gate_up_weight)):
            gate_up = "skinny"
        elif self.gate_up_weight.numel() * 2 >= 100e6 and ops.wide_gemm_takes_rows(ops.EPI_SWIGLU, rows, self.gate_up_weight):
            gate_up = "wide"
        return gate_up, ops.residual_product_way(rows, self.down_weight)

    def fused_takes(self, ctx) -> bool:
        return (ctx.dtype == torch.bfloat16 and ctx.attention == "auto" and self.inter % 8 == 0
                and ctx.n_tokens <= ops.WIDE_MAX_ROWS and self._ways(ctx) != ("unfused", "unfused"))

    def fused_forward(self, hidden, rms, ctx, delta=None):
        gate_up, down = self._ways(ctx)
        act = torch.empty((hidden.shape[0], self.inter), dtype=torch.bfloat16, device=hidden.device)
        if gate_up == "skinny":
            if delta is not None:
                ops.residual_add(hidden, delta)
            ops.skinny_gemm(ops.EPI_SWIGLU, self.gate_up_weight, hidden=hidden, norm_weight=rms[0], eps=rms[1], out=act)
        else:
            x = torch.empty(hidden.shape, dtype=torch.bfloat16, device=hidden.device)
            ops.add_rms_norm(hidden, delta, rms[0], rms[1], x)   # the norm kernel adds the pending delta on its way
            if gate_up == "wide":
                ops.wide_gemm(ops.EPI_SWIGLU, self.gate_up_weight, x=x, out=act, err=ctx.err)
            else:
                ops.swiglu(ops.linear(x, self.gate_up_weight), act)
        if down == "skinny":
            ops.skinny_gemm(ops.EPI_RESIDUAL, self.down_weight, x=act, residual=hidden)
        elif down == "wide":
            ops.wide_gemm(ops.EPI_RESIDUAL, self.down_weight, x=act, residual=hidden, err=ctx.err)
        else:
            ops.residual_add(hidden, ops.linear(act, self.down_weight))


register_part("feed_forward", "swiglu", SwiGlu)
