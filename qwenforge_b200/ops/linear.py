"""Dense projections: y = x W^T (+ b).

float32 runs this library's own FFMA kernel (true 32-bit, a fixed order of additions for
every output element). bfloat16 calls the cuBLAS matrix product through torch, the same
library call the reference makes for its projections (student_engine.py:563, :664, :666,
:727, :736), until the tensor-core kernel of this library covers the shape.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import kernels

# Plain products of 128 or more token rows can run on this library's own tcgen05 kernel (`csrc/tc_gemm.cu`) instead of
# the cuBLAS call. Off by default: measured on a B200 at 2048 x 9728 x 896 its persistent form reaches 800 TFLOP/s where
# cuBLAS reaches 1,140 (at 2048 x 37888 x 3584: 1,215 against 1,620). The gate/up product with the gate in its epilogue
# does not wait for this switch: it is the faster way wherever the persistent kernel runs (`parts/swiglu.py`).
_own_tensor_core_products = False
OWN_PRODUCT_MIN_ROWS = 128


def use_own_tensor_core_products(on: bool) -> None:
    global _own_tensor_core_products
    _own_tensor_core_products = bool(on)


def own_tensor_core_products(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether x @ weight.T is to run on the library's own tcgen05 kernel."""
    return (_own_tensor_core_products and x.dtype == torch.bfloat16 and x.shape[0] >= OWN_PRODUCT_MIN_ROWS
            and weight.shape[0] % 8 == 0 and kernels.tc_gemm_takes(x, weight))


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """x [M, K], weight [N, K] -> [M, N]. `out_dtype=torch.float32` asks a bfloat16 product for
    float32 results (accumulated in float32 and not rounded to bfloat16), as the logits need."""
    if not x.is_cuda:
        raise kernels.KernelError(f"linear: input on {x.device}; this library computes on CUDA devices only")
    m, n = x.shape[0], weight.shape[0]
    if x.dtype == torch.float32:
        if out is None:
            out = torch.empty((m, n), device=x.device, dtype=torch.float32)
        kernels.gemm_f32(x, weight, bias, out)
        return out
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise kernels.KernelError(f"linear: dtypes {x.dtype} x {weight.dtype} are not supported")
    if out_dtype != torch.float32 and bias is None and own_tensor_core_products(x, weight):
        if out is None:
            out = torch.empty((m, n), device=x.device, dtype=torch.bfloat16)
        kernels.tc_gemm(kernels.TC_PLAIN, x, weight, out)
        return out
    if out_dtype == torch.float32:
        result = torch.mm(x, weight.t(), out_dtype=torch.float32)
        if bias is not None:
            result += bias.float()
        if out is not None:
            out.copy_(result)
            return out
        return result
    if out is not None:
        if bias is None:
            torch.mm(x, weight.t(), out=out)
        else:
            torch.addmm(bias, x, weight.t(), out=out)
        return out
    return torch.nn.functional.linear(x, weight, bias)
