"""The generation loop above the step function.

Requests are served in batches of `batch_size`, in order, one batch after another (the reference
chunks its prompts the same way, student_engine.py:1395-1398). The sequences of a batch start
together: ONE step runs all their prompts, of unequal lengths and without padding; the token chosen
from each prompt's last position is output token 0 (:1320), and each further step feeds every live
sequence its latest token (:1120-1126), so `max_new_tokens` tokens cost one prompt step and
`max_new_tokens - 1` single-token steps.

Unlike the reference, whose batches end together after exactly `max_new_tokens` steps and which
ignores end-of-sequence tokens (:1126, scripts/run_inference_benchmark.py:596-597), a sequence here
ends on its own: when it produces a stop token (kept as its last output token) or when its budget is
spent. It leaves the batch at once and its cache slot is given back; the next batch takes the
freed slots again. `ignore_eos=True` restores the reference's fixed-length behaviour.

The loop is written against a small `Stepper` interface, so its decisions can be tested without a GPU.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Optional, Protocol, Sequence


class Stepper(Protocol):
    """What the loop needs from the model and its cache."""

    max_positions: int

    def open(self) -> int: ...
    def close(self, slot: int) -> None: ...
    def reserve(self, slot_totals: Sequence[tuple[int, int]]) -> None: ...
    def step_and_choose(self, entries: Sequence[tuple[int, Sequence[int]]], seq_ids: Sequence[int],
                        steps: Sequence[int]) -> list[int]: ...

    # Optional: a stepper may also offer `open_decode_session(rows, stop_token_ids)`, with rows of
    # (slot, latest token, sequence id, tokens generated so far, budget). It returns None, or an object whose
    # `run(n)` performs up to n single-token steps for all rows without the host in between and returns, per
    # step, each row's produced token (-1 once the row has ended, by the same rules as the loop's).


@dataclass
class SequenceResult:
    tokens: list = field(default_factory=list)
    finish_reason: str = ""  # "stop" | "length"


@dataclass
class _Live:
    index: int          # position of the request in the call (also its sampling key)
    slot: int
    budget: int
    result: SequenceResult


class GenerationLoop:
    def __init__(self, stepper: Stepper, stop_token_ids: Sequence[int] = (), ignore_eos: bool = False,
                 bos_token_id: Optional[int] = None):
        self.stepper = stepper
        self.stop_token_ids = frozenset(int(t) for t in stop_token_ids)
        self.ignore_eos = ignore_eos
        self.bos_token_id = bos_token_id
        self.steps_run = 0            # decode steps of the last call, for callers that measure
        self.prompt_steps_run = 0
        self.decode_seconds = 0.0     # host time of those decode steps (each ends with the tokens on the host)
        self.decoded_tokens = 0

    def _stops(self, token: int) -> bool:
        return not self.ignore_eos and token in self.stop_token_ids

    def run(self, prompts: Sequence[Sequence[int]], max_new_tokens, batch_size: int = 1) -> list[SequenceResult]:
        """prompts: token ids per request; max_new_tokens: one budget for all or one per request."""
        n = len(prompts)
        budgets = [int(max_new_tokens)] * n if isinstance(max_new_tokens, int) else [int(b) for b in max_new_tokens]
        if len(budgets) != n:
            raise ValueError("max_new_tokens must be one number or one per prompt")
        results = [SequenceResult() for _ in range(n)]
        self.steps_run = self.prompt_steps_run = self.decoded_tokens = 0
        self.decode_seconds = 0.0
        size = max(int(batch_size), 1)
        for begin in range(0, n, size):
            self._run_batch(list(range(begin, min(begin + size, n))), prompts, budgets, results)
        return results

    def _run_batch(self, indices, prompts, budgets, results) -> None:
        stepper = self.stepper
        batch = []
        for i in indices:
            tokens = list(prompts[i])
            if not tokens:  # the reference feeds one BOS to an empty prompt (student_engine.py:1244-1253)
                if self.bos_token_id is None:
                    raise ValueError("Cannot generate from an empty prompt without a BOS token")
                tokens = [self.bos_token_id]
            if budgets[i] <= 0:
                results[i].finish_reason = "length"
                continue
            if len(tokens) + budgets[i] > stepper.max_positions:
                raise ValueError(f"Requested sequence length {len(tokens) + budgets[i]} "
                                 f"exceeds model limit {stepper.max_positions}")
            batch.append((i, tokens))
        if not batch:
            return
        live: list[_Live] = []
        try:
            for i, tokens in batch:
                live.append(_Live(i, stepper.open(), budgets[i], results[i]))
            # room for every sequence's whole future, so that no later step can run out of cache
            stepper.reserve([(s.slot, len(tokens) + s.budget - 1) for s, (_, tokens) in zip(live, batch)])
            chosen = stepper.step_and_choose([(s.slot, tokens) for s, (_, tokens) in zip(live, batch)],
                                             [s.index for s in live], [0] * len(live))
            self.prompt_steps_run += 1
            live = self._take(live, chosen)
            started = time.perf_counter()
            session = None
            if live and hasattr(stepper, "open_decode_session"):
                session = stepper.open_decode_session(
                    [(s.slot, s.result.tokens[-1], s.index, len(s.result.tokens), s.budget) for s in live],
                    () if self.ignore_eos else tuple(self.stop_token_ids))
            if session is not None:
                live = self._run_session(session, live)
            while live:
                chosen = stepper.step_and_choose([(s.slot, [s.result.tokens[-1]]) for s in live],
                                                 [s.index for s in live], [len(s.result.tokens) for s in live])
                self.steps_run += 1
                self.decoded_tokens += len(live)
                live = self._take(live, chosen)
            self.decode_seconds += time.perf_counter() - started
        finally:
            for s in live:  # only after an exception: normal ends have closed their slots already
                stepper.close(s.slot)

    def _run_session(self, session, live: list) -> list:
        """Decode with a host-free session: read the produced tokens chunk by chunk and apply the same decisions."""
        rows = list(live)
        while live:
            remaining = max(s.budget - len(s.result.tokens) for s in live)
            for step_tokens in session.run(remaining):
                if not live:
                    break
                chosen = [step_tokens[rows.index(s)] for s in live]
                if any(t < 0 for t in chosen):
                    raise RuntimeError("decode session and generation loop disagree on which sequences are live")
                self.steps_run += 1
                self.decoded_tokens += len(live)
                live = self._take(live, chosen)
        return live

    def _take(self, live: list, chosen: Sequence[int]) -> list:
        """Append each sequence's new token; sequences that end leave the batch and free their slot."""
        still = []
        for s, token in zip(live, chosen):
            s.result.tokens.append(int(token))
            if self._stops(int(token)):
                s.result.finish_reason = "stop"
            elif len(s.result.tokens) >= s.budget:
                s.result.finish_reason = "length"
            if s.result.finish_reason:
                self.stepper.close(s.slot)
            else:
                still.append(s)
        return still
