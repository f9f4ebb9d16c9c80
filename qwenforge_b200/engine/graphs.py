"""Decode steps replayed from CUDA graphs, without the host between steps.

The reference captures its whole decode step once per (batch, cache capacity) and replays it, patching a write
index, a position and a mask slot from the host before every replay (student_engine.py:984-1133). Here everything
that changes from step to step lives on the device: the rows' input tokens, positions, step counts and slots are
static buffers that the step's own last kernel (`decode_advance`) updates, and the page tables already cover each
sequence's whole budget, so a replay needs no host work at all and the host reads the produced tokens only once
per chunk of steps.

A captured graph is keyed by (rows, bound on the longest sequence, sampling temperature and seed): the bound fixes
how the decode attention splits its key range, the sampling scalars are arguments of the sampling kernel. Graphs
are kept and replayed by later batches of the same key (the reference's registry, :1081-1118). Rows that end early
stay in the launch as padding entries (slot -1), which touch no cache and change no result.
"""
from __future__ import annotations

import contextlib
import dataclasses
import gc
from typing import Optional

import numpy as np
import torch

from .. import ops
from ..sampling import Sampler
from .step import StepContext, pack_step

MAX_STOP_IDS = 8
CHUNK_STEPS = 32


@contextlib.contextmanager
def capturing(graph: torch.cuda.CUDAGraph, stream: torch.cuda.Stream, pool=None):
    """`torch.cuda.graph` with Python's cycle collector held off meanwhile. Destroying an older graph is a call that
    CUDA forbids while any stream captures, and it ends the capture with an error; an older graph that sits in a
    reference cycle is destroyed whenever the collector happens to run, which may be in the middle of this capture.
    So what is collectable goes first, and the collector waits until the capture has ended."""
    gc.collect()
    was_enabled = gc.isenabled()
    gc.disable()
    try:
        with torch.cuda.graph(graph, stream=stream, pool=pool):
            yield
    finally:
        if was_enabled:
            gc.enable()


def length_bound(n: int) -> int:
    """The next power of two >= n (at least 256): sequences of similar length share a graph."""
    bound = 256
    while bound < n:
        bound *= 2
    return bound


class DecodeGraph:
    """Static buffers and the captured step for `rows` sequences."""

    def __init__(self, model, cache, rows: int, max_len: int, sampler: Sampler):
        device = model.device
        self.model, self.cache, self.rows, self.sampler = model, cache, rows, sampler
        i32 = dict(dtype=torch.int32, device=device)
        self.token_ids = torch.zeros(rows, **i32)
        self.tok_pos = torch.zeros(rows, **i32)
        self.slots = torch.full((rows,), -1, **i32)
        self.steps = torch.zeros(rows, **i32)
        self.budgets = torch.zeros(rows, **i32)
        self.seq_ids = torch.zeros(rows, dtype=torch.int64, device=device)
        self.stop_ids = torch.full((MAX_STOP_IDS,), -1, **i32)
        self.sampled = torch.zeros(rows, **i32)
        self.out_tokens = torch.full((CHUNK_STEPS, rows), -1, **i32)
        self.cursor = torch.zeros(1, **i32)
        self.n_stop = 0
        arange = torch.arange(rows + 1, **i32)
        self.ctx = StepContext(
            n_seqs=rows, n_tokens=rows, max_q_len=1, max_kv_len=max_len, token_ids=self.token_ids,
            tok_seq=arange[:rows].clone(), tok_pos=self.tok_pos, slots=self.slots, cu_q=arange,
            want_rows=arange[:rows].clone(), err=model.err, dtype=model.dtype, attention=model.attention,
            decode_scratch=ops.DecodeScratch(device))  # the graph's own: its addresses are baked into the capture
        self.sample_scratch = ops.SampleScratch()
        # Where the embedding is a plain lookup, the kernel that advances the rows' state also embeds their next tokens,
        # and a step starts at its first layer.
        lookup = getattr(model.embedding, "lookup_table", None)
        self.table = lookup() if lookup is not None else None
        if self.table is not None:
            self.ctx.embedded = torch.zeros((rows, self.table.shape[1]), dtype=torch.float32, device=device)
            self.ticket = torch.zeros(1, **i32)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.kernels_per_step = 0
        self.last_logits: Optional[torch.Tensor] = None  # float32 [rows, vocab] of the newest replayed step

    def _one_step(self) -> None:
        logits = self.model.forward(self.ctx, self.cache)
        self.last_logits = logits  # inside a capture this is the graph's own buffer: every replay refills it
        self.sampler(logits, self.seq_ids, self.steps, out=self.sampled, scratch=self.sample_scratch)
        if self.table is not None:
            ops.decode_advance_embed(self.sampled, self.token_ids, self.tok_pos, self.slots, self.steps, self.budgets,
                                     self.stop_ids, MAX_STOP_IDS, self.out_tokens, self.cursor, self.table,
                                     self.ctx.embedded, self.ticket, self.model.err)
        else:
            ops.decode_advance(self.sampled, self.token_ids, self.tok_pos, self.slots, self.steps, self.budgets,
                               self.stop_ids, MAX_STOP_IDS, self.out_tokens, self.cursor)

    def load(self, slots, tokens, positions, steps, budgets, seq_ids, stop_ids) -> None:
        """Set the rows' state (rows beyond the given ones are padding)."""
        pad = self.rows - len(slots)
        packed = torch.tensor([list(tokens) + [0] * pad, list(positions) + [0] * pad, list(slots) + [-1] * pad,
                               list(steps) + [0] * pad, list(budgets) + [0] * pad], dtype=torch.int32)
        packed = packed.to(self.token_ids.device)
        self.token_ids.copy_(packed[0])
        self.tok_pos.copy_(packed[1])
        self.slots.copy_(packed[2])
        self.steps.copy_(packed[3])
        self.budgets.copy_(packed[4])
        self.seq_ids.copy_(torch.tensor(list(seq_ids) + [0] * pad, dtype=torch.int64).to(self.seq_ids.device))
        stops = list(stop_ids)[:MAX_STOP_IDS]
        self.stop_ids.copy_(torch.tensor(stops + [-1] * (MAX_STOP_IDS - len(stops)), dtype=torch.int32))
        if self.table is not None:   # the first step's rows; every later step's come from the step before it
            ops.embed_gather(self.token_ids, self.table, self.ctx.embedded, self.model.err)

    def capture(self) -> None:
        """Two eager steps on a side stream (they size every scratch buffer), then the capture. The rows are all
        padding meanwhile (slot -1), so neither touches the cache or the rows' state."""
        saved = self.slots.clone()
        self.slots.fill_(-1)
        stream = torch.cuda.Stream(device=self.model.device)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for _ in range(2):
                self._one_step()
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()
        before = ops.kernels.launches
        graph = torch.cuda.CUDAGraph()
        with capturing(graph, stream):
            self._one_step()
        self.kernels_per_step = ops.kernels.launches - before
        self.graph = graph
        self.cursor.zero_()
        self.slots.copy_(saved)

    def enqueue(self, n_steps: int) -> int:
        """Put `n_steps` (at most CHUNK_STEPS) steps on the stream; returns how many. Their tokens overwrite those of the
        chunk before: collect that one first."""
        n_steps = min(n_steps, CHUNK_STEPS)
        self.cursor.zero_()
        for _ in range(n_steps):
            self.graph.replay()
        ops.kernels.launches += self.kernels_per_step * n_steps
        return n_steps

    def collect(self, n_steps: int) -> tuple:
        """Wait for the enqueued chunk of `n_steps` steps and read it back in ONE copy: per step the rows' produced
        tokens (-1: none), the most steps any row still has to go (0: every row has ended), the device error word."""
        rows = self.rows
        left = torch.where(self.slots >= 0, self.budgets - self.steps, torch.zeros_like(self.steps))
        packed = torch.cat((self.out_tokens[:n_steps].flatten(), left, self.model.err)).tolist()
        tokens = [packed[i * rows:(i + 1) * rows] for i in range(n_steps)]
        return tokens, max(packed[n_steps * rows:n_steps * rows + rows], default=0), packed[-1]

    def run(self, n_steps: int) -> list:
        """Replay `n_steps` (<= CHUNK_STEPS) steps; returns per step the rows' produced tokens (-1: none)."""
        return self.collect(self.enqueue(n_steps))[0]


class GraphDecoder:
    """Keeps captured decode graphs of one model and cache, newest last; old ones are dropped beyond `keep`."""

    def __init__(self, model, cache, keep: int = 8):
        self.model, self.cache, self.keep = model, cache, keep
        self.graphs: dict = {}

    @staticmethod
    def supported(model) -> bool:
        return all(getattr(part, "graph_safe", True) for part in model.parts())

    def get(self, rows: int, max_len: int, sampler: Sampler) -> DecodeGraph:
        key = (rows, length_bound(max_len), sampler.params.temperature, sampler.params.seed)
        graph = self.graphs.pop(key, None)
        if graph is None:
            graph = DecodeGraph(self.model, self.cache, rows, key[1], sampler)
            graph.capture()
        self.graphs[key] = graph
        while len(self.graphs) > self.keep:
            self.graphs.pop(next(iter(self.graphs)))
        return graph


class PrefillGraphs:
    """Steps of whole prompts or continuations replayed from CUDA graphs when their shape comes back.

    A step of a few thousand tokens of a small model is bound by the host: two hundred launches take longer to issue
    than to run. What fixes those launches is the step's shape (tokens, entries, longest entry, wanted rows) and
    the cache it works on; everything else (token ids, positions, slots, page tables) is data in device buffers.
    So that prompts of any length meet a shape that came before, a step is first brought to a rounded shape: one
    padding entry (slot -1: computed, touches no cache, changes no result) fills its token count up to the next
    multiple of a granule (64 tokens up to 512, then 128, 256 and 512: at most an eighth more work), and the longest
    entry is rounded up likewise (blocks of rows that no entry has end at once). A step whose token count is a
    multiple of the granule already gets no padding entry. The second step of a rounded shape is captured, with its
    integers in a buffer of the graph's own; every later one copies its integers there and replays. Steps of more
    than `MAX_TOKENS` tokens are bound by the GPU and are left alone, as are single-token steps (the decode graphs'
    business). The newest `keep` graphs are kept; they share one memory pool, since no two run at the same time.
    """

    MAX_TOKENS = 8192

    def __init__(self, model, keep: int = 24):
        self.model, self.keep = model, keep
        self.seen: dict = {}     # shape -> how often it came
        self.graphs: dict = {}   # shape -> (graph, integer buffer, logits); newest last
        self.pool = None
        self.replays = 0

    def takes(self, step) -> bool:
        return 1 < step.max_q_len and step.n_tokens <= self.MAX_TOKENS

    @staticmethod
    def granule(n_tokens: int) -> int:
        return 64 if n_tokens <= 512 else 128 if n_tokens <= 2048 else 256 if n_tokens <= 4096 else 512

    @classmethod
    def rounded(cls, step, triples, want):
        """The step brought to its rounded shape (see the class): the same entries and wanted places, then one padding
        entry if the token count is no multiple of the granule; the bounds on the longest entry rounded up."""
        g = cls.granule(step.n_tokens)
        pad = -step.n_tokens % g
        if pad:
            triples = list(triples) + [(-1, 0, np.zeros(pad, dtype=np.int32))]
            want = None if want is None else list(want) + [[]]
            step = pack_step(triples, want)
        up = lambda n: -(-n // g) * g
        return dataclasses.replace(step, max_q_len=up(step.max_q_len), max_kv_len=up(step.max_kv_len))

    def run(self, cache, step, triples, want) -> Optional[torch.Tensor]:
        """The step's logits by replay, or None if its rounded shape has no graph yet (the caller then runs the step
        as it is; the second time a rounded shape comes it is captured here and its logits are returned)."""
        step = self.rounded(step, triples, want)
        key = (cache.serial,) + step.shape_key
        held = self.graphs.pop(key, None)
        if held is None:
            self.seen[key] = self.seen.get(key, 0) + 1
            if len(self.seen) > 4096:
                self.seen.clear()
            if self.seen[key] < 2:
                return None
            try:
                held = self._capture(cache, step)
            except RuntimeError as exc:  # e.g. no memory for the graph's pool: this shape goes on launch by launch
                import sys
                print(f"[qwenforge_b200] a prompt step of shape {step.shape_key} could not be captured ({exc}); "
                      "it runs launch by launch", file=sys.stderr, flush=True)
                self.seen[key] = -(1 << 30)
                return None
        self.graphs[key] = held  # newest last
        while len(self.graphs) > self.keep:
            self.graphs.pop(next(iter(self.graphs)))
        graph, integers, logits, launches = held
        # from pageable memory the copy is complete when the call returns, so the host array may go
        integers.copy_(torch.from_numpy(step.packed))
        graph.replay()
        self.replays += 1
        ops.kernels.launches += launches
        return None if logits is None else logits.clone()

    def _capture(self, cache, step):
        from .step import context_of
        model = self.model
        integers = torch.zeros(step.packed.size, dtype=torch.int32, device=model.device)
        integers.copy_(torch.from_numpy(step.packed))
        ctx = context_of(step, integers, model.err, model.dtype, model.attention, model.decode_scratch)
        ctx.host_slots = ctx.host_starts = ctx.host_q_lens = None  # a replay's differ: no part may plan on them
        stream = torch.cuda.Stream(device=model.device)
        stream.wait_stream(torch.cuda.current_stream())
        torch.cuda.synchronize()
        before = ops.kernels.launches
        graph = torch.cuda.CUDAGraph()
        with capturing(graph, stream, self.pool):
            logits = model.forward(ctx, cache)
        if self.pool is None:
            self.pool = graph.pool()
        return graph, integers, logits, ops.kernels.launches - before
