"""Next-token choice. The reference chooses greedily only (student_engine.py:1320, :982, :1158:
argmax of the last position's logits) and accepts a seed that no stochastic operation reads
(:316, :425-427). This library adds temperature sampling: temperature 0 is the reference's greedy
choice (lowest id on ties), temperature > 0 draws from softmax(logits / temperature) with the
Gumbel-max kernel, keyed by (seed, sequence id, number of tokens the sequence has generated), so a
sequence's tokens do not depend on which batch it runs in."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import ops


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    seed: int = 0

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")


class Sampler:
    def __init__(self, params: SamplingParams = SamplingParams()):
        self.params = params

    @property
    def greedy(self) -> bool:
        return self.params.temperature <= 0.0

    def __call__(self, logits: torch.Tensor, seq_ids: Optional[torch.Tensor] = None,
                 steps: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None, scratch=None) -> torch.Tensor:
        """logits float32 [rows, vocab] -> int32 [rows]; seq_ids int64 [rows] and steps int32 [rows] when sampling."""
        if out is None:
            out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
        ops.sample(logits, self.params.temperature, self.params.seed, seq_ids, steps, out, scratch)
        return out
