"""Token embedding into the float32 residual stream (student_engine.py:690) and the output head
(:733-736: logits = normed W^T, no bias; W is the embedding table when the model ties them, :359)."""
from __future__ import annotations

import torch

from .. import ops
from .base import Embedding, Part, TensorSpec
from .registry import register_part


class TokenEmbedding(Embedding):
    """params: vocab_size, width. tensors: weight [vocab_size, width]."""

    def __init__(self, spec):
        super().__init__(spec)
        self.vocab = int(self.params["vocab_size"])
        self.width = int(self.params["width"])
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.file_name("weight"), (self.vocab, self.width))]

    def kernel_libraries(self, dtype):
        return {"embed"}

    def bind(self, tensors, dtype, device):
        self.weight = tensors[self.file_name("weight")]

    def lookup_table(self):
        return self.weight

    def forward(self, token_ids: torch.Tensor, ctx) -> torch.Tensor:
        hidden = torch.empty((token_ids.numel(), self.width), dtype=torch.float32, device=token_ids.device)
        ops.embed_gather(token_ids, self.weight, hidden, ctx.err)
        return hidden


class LinearHead(Part):
    """params: vocab_size, width, tied. tensors: weight [vocab_size, width] (the embedding's tensor when tied), and
    optionally weight_fallback: the tensor that serves when the files hold no `weight` (the reference takes the
    embedding table whenever lm_head.weight is absent, student_engine.py:359). Returns float32 logits in both precisions."""

    def __init__(self, spec):
        super().__init__(spec)
        self.vocab = int(self.params["vocab_size"])
        self.width = int(self.params["width"])
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.file_name("weight"), (self.vocab, self.width),
                           fallback=self.spec.tensors.get("weight_fallback"))]

    def kernel_libraries(self, dtype):
        return {"gemm_f32"} if dtype == torch.float32 else set()

    def bind(self, tensors, dtype, device):
        self.weight = tensors[self.file_name("weight")]

    def step_weights(self):
        return [self.weight]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, self.weight, None, out_dtype=torch.float32)


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "linear_head", LinearHead)
