"""What one step runs: a batch of sequences that either all start (whole prompts, unequal lengths)
or all go on (one or more further tokens each), laid out without padding.

Token t of the flat batch belongs to batch entry `tok_seq[t]` and stands at absolute position
`tok_pos[t]` of its sequence; entry s owns tokens `cu_q[s] .. cu_q[s+1]-1` and the cache slot
`slots[s]` (-1 marks a padding entry: it is computed, touches no cache and changes no result).
All of it goes to the device in one copy.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch


@dataclass
class StepContext:
    n_seqs: int
    n_tokens: int
    max_q_len: int
    max_kv_len: int                  # upper bound of any sequence's length after this step
    token_ids: torch.Tensor          # int32 [T]
    tok_seq: torch.Tensor            # int32 [T]
    tok_pos: torch.Tensor            # int32 [T]
    slots: torch.Tensor              # int32 [n]
    cu_q: torch.Tensor               # int32 [n + 1]
    want_rows: Optional[torch.Tensor]  # int32 [R] flat token indices whose logits are wanted
    err: torch.Tensor                # int32 [1] device error word
    dtype: torch.dtype
    attention: str = "auto"          # "auto": fastest kernel that takes the shape; "generic": the SIMT kernel
    decode_scratch: Optional[object] = None   # ops.DecodeScratch shared by the model's attention layers
    # per-token side inputs named by whoever feeds the step, [T, ...] on the device: what a part needs beyond a
    # token's index in its sequence (positions on several axes, token types). `tok_pos` stays the index that
    # orders the cache and the causal mask.
    extras: Optional[dict] = None
    # the step's tokens already embedded into the float32 stream [T, W] (a decode graph's state kernel leaves the next
    # step's rows there); the model then starts at its first layer
    embedded: Optional[torch.Tensor] = None
    # what the parts of one step share: the model empties it before every run of its schedule; a part keeps there
    # what it works out once per step for all layers of its kind (key: a tuple that starts with the part's own name)
    step_memo: Optional[dict] = None
    # host copies, for parts that plan on the host (absent when a captured graph replays the step)
    host_slots: Optional[list] = None
    host_starts: Optional[list] = None
    host_q_lens: Optional[list] = None

    @property
    def is_decode(self) -> bool:
        return self.max_q_len == 1


@dataclass
class PackedStep:
    """A step's integers on the host, ready for ONE copy: ids | tok_seq | tok_pos | slots | cu_q | rows."""
    packed: np.ndarray
    n_seqs: int
    n_tokens: int
    n_rows: int
    max_q_len: int
    max_kv_len: int
    host_slots: list
    host_starts: list
    host_q_lens: list

    @property
    def shape_key(self) -> tuple:
        """What fixes the launches of a step of whole prompts or continuations (not the values they work on)."""
        return (self.n_tokens, self.n_seqs, self.max_q_len, self.n_rows)


def pack_step(entries: Sequence[tuple[int, int, Sequence[int]]], want: Optional[Sequence[Sequence[int]]]) -> PackedStep:
    """entries: (slot, start_position, token ids) per batch entry; want: per entry, the places among its
    tokens whose logits are wanted (None: the last token of every entry with a real slot)."""
    id_parts, seq_parts, pos_parts = [], [], []
    slots: list[int] = []
    cu_q = [0]
    rows: list[int] = []
    for s, (slot, start, tokens) in enumerate(entries):
        q = len(tokens)
        if q == 0:
            raise ValueError(f"step: entry {s} brings no tokens")
        base = cu_q[-1]
        id_parts.append(np.asarray(tokens, dtype=np.int32))
        seq_parts.append(np.full(q, s, dtype=np.int32))
        pos_parts.append(np.arange(start, start + q, dtype=np.int32))
        slots.append(slot)
        cu_q.append(base + q)
        if want is None:
            if slot >= 0:
                rows.append(base + q - 1)
        else:
            for place in want[s]:
                if not 0 <= place < q:
                    raise ValueError(f"step: entry {s} wants place {place} of {q} tokens")
                rows.append(base + place)
    packed = np.concatenate(id_parts + seq_parts + pos_parts + [np.asarray(slots + cu_q + rows, dtype=np.int32)])
    return PackedStep(packed=packed, n_seqs=len(entries), n_tokens=cu_q[-1], n_rows=len(rows),
                      max_q_len=max(len(e[2]) for e in entries), max_kv_len=max(e[1] + len(e[2]) for e in entries),
                      host_slots=list(slots), host_starts=[e[1] for e in entries], host_q_lens=[len(e[2]) for e in entries])


def context_of(step: PackedStep, dev: torch.Tensor, err: torch.Tensor, dtype: torch.dtype, attention: str = "auto",
               decode_scratch=None) -> StepContext:
    """The context whose tensors are views of `dev`, a device copy of `step.packed` (or a buffer that will hold one)."""
    o = 0

    def take(count):
        nonlocal o
        piece = dev[o:o + count]
        o += count
        return piece

    n, total = step.n_seqs, step.n_tokens
    return StepContext(
        n_seqs=n, n_tokens=total, max_q_len=step.max_q_len, max_kv_len=step.max_kv_len,
        token_ids=take(total), tok_seq=take(total), tok_pos=take(total), slots=take(n), cu_q=take(n + 1),
        want_rows=take(step.n_rows) if step.n_rows else None, err=err, dtype=dtype, attention=attention,
        decode_scratch=decode_scratch,
        host_slots=step.host_slots, host_starts=step.host_starts, host_q_lens=step.host_q_lens,
    )


def build_context(entries: Sequence[tuple[int, int, Sequence[int]]], want: Optional[Sequence[Sequence[int]]],
                  err: torch.Tensor, dtype: torch.dtype, device, attention: str = "auto",
                  decode_scratch=None) -> StepContext:
    """Pack the step on the host, copy it to the device in one copy, and view the copy as the step's tensors."""
    step = pack_step(entries, want)
    # from pageable memory the copy is complete when the call returns, so the host array may go
    dev = torch.from_numpy(step.packed).to(device)
    return context_of(step, dev, err, dtype, attention, decode_scratch)
