"""Interfaces of the parts a layer is put together from.

A part is built from a `PartSpec` alone: its sizes and constants are the spec's `params`,
the tensors it owns are named by the spec's `tensors`. No part knows which model it is in,
which layer it is, or what the other parts of its layer are.

Life of a part:
  1. `Part(spec)`           metadata only, no device memory
  2. `tensor_specs()`       what it wants from the weight files (name, shape, how to draw it at random)
  3. `kernel_libraries(dt)` which kernel libraries it will call for activation dtype `dt`
  4. `bind(tensors, dt, device)`  take its tensors (already on the device and in their kept dtype) and
                            arrange them as its kernels want them (fused, concatenated)
  5. `forward(...)`         per step

Interfaces by role (T = tokens of the step, W = model width):
  Norm           forward(hidden f32 [T, W] (updated in place), delta [T, W] | None) -> normed [T, W]
                 computes hidden += delta, then normalises.
  Mixer          cache_need() -> KvNeed | StateNeed | None
                 forward(x [T, W], ctx, site, writes_cache) -> delta [T, W]
                 `site` is the cache view of the schedule entry being run (or of the entry it
                 reads from when `writes_cache` is false).
  FeedForward    forward(x [T, W], ctx) -> delta [T, W]
  PositionEncoding
                 fused_rotary() -> (inv_freq f32 [R/2], R) | None   what a mixer's fused kernel may apply itself
                 apply(q [T, NH, D], k [T, KVH, D], ctx) -> None    in place, when there is no fused form
  Block          forward(hidden, delta, ctx, site, writes_cache) -> delta
                 arranges norms, mixer and feed-forward around the residual stream `hidden`.
Mixers and feed-forwards may also offer a form for steps of a few tokens that works on the stream in place
(`fused_takes`, `fused_forward`): it adds the pending delta of the part before, applies the preceding RMSNorm in its own
first kernel and adds its result to `hidden`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Mapping, Optional

import torch

from ..config.spec import PartSpec


@dataclass(frozen=True)
class TensorSpec:
    """One tensor of the weight files.

    init  how the random-weights mode draws it: "matrix" N(0, 0.02), "bias" N(0, 0.02), "norm" 1 + N(0, 0.1)
    keep  "compute": kept in the activation dtype (bfloat16, or float32 on the 32-bit path)
          "stored":  kept as the file stores it if that is a 32-bit float, else as "compute"
          "int32":   an integer table, kept as int32
    fallback  another tensor name that stands in when the files do not hold `name` (a head that
              shares the embedding table in files that say nothing about tying)
    """
    name: str
    shape: tuple
    init: str = "matrix"
    keep: str = "compute"
    fallback: Optional[str] = None


class Part:
    kind = ""
    # False for a part whose forward needs the step's host-side lists (ctx.host_*): a model with such a part
    # decodes step by step instead of replaying captured graphs
    graph_safe = True

    def __init__(self, spec: PartSpec):
        self.spec = spec
        self.params = dict(spec.params)

    def file_name(self, logical: str) -> str:
        try:
            return self.spec.tensors[logical]
        except KeyError:
            raise KeyError(f"part {self.kind!r}: its spec names no tensor for {logical!r}") from None

    def tensor_specs(self) -> list[TensorSpec]:
        return []

    def kernel_libraries(self, dtype: torch.dtype) -> set[str]:
        return set()

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype, device) -> None:
        pass

    def sub_parts(self) -> list["Part"]:
        return []

    def step_weights(self) -> list:
        """The bound tensors that every step reads in full (for the measurement's byte counts); tables that a step
        only gathers rows from are not among them."""
        return []


class Embedding(Part):
    def forward(self, token_ids: torch.Tensor, ctx) -> torch.Tensor:
        """The float32 residual stream [T, width] of the step's token ids."""
        raise NotImplementedError

    def lookup_table(self):
        """The table [vocab, width] if this embedding is a plain row lookup (row id -> stream row, nothing added or
        scaled), which the kernel that advances a decode graph's state may then do for the next step; else None."""
        return None


class Norm(Part):
    def forward(self, hidden: torch.Tensor, delta: Optional[torch.Tensor]) -> torch.Tensor:
        raise NotImplementedError

    def fused_rms(self):
        """(weight, eps) if this norm is a plain RMSNorm that a following kernel may apply in its prologue, else None."""
        return None


class Mixer(Part):
    def cache_need(self):
        return None

    def forward(self, x: torch.Tensor, ctx, site, writes_cache: bool) -> torch.Tensor:
        raise NotImplementedError

    # Optional fast form for steps of a few tokens: the part adds the pending `delta` (if any) to the residual stream,
    # applies the preceding RMSNorm itself and adds its output to the stream in place
    # (hidden += delta; hidden += mixer(rmsnorm(hidden))). A block uses it when `fused_takes(ctx)` is true and its norm
    # has a `fused_rms()` form.
    def fused_takes(self, ctx) -> bool:
        return False

    def fused_forward(self, hidden: torch.Tensor, rms, ctx, site, writes_cache: bool, delta=None) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError

    def fused_takes(self, ctx) -> bool:
        return False

    def fused_forward(self, hidden: torch.Tensor, rms, ctx, delta=None) -> None:
        raise NotImplementedError


class PositionEncoding(Part):
    def fused_rotary(self):
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor, ctx) -> None:
        raise NotImplementedError
