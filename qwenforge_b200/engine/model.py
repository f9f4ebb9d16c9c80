"""The model runtime: parts built from a `ModelSpec`, a schedule of layer runs, and ONE step function.

`Model.step(cache, entries, want)` is everything between a request's tokens and its logits:
  embed the step's tokens -> run the schedule (each entry: a block, with its own cache view or an
  earlier entry's) -> gather the wanted rows -> final norm -> head -> float32 logits [wanted, vocab].
It runs only the tokens it is given, as one batch, from the cache that earlier steps left.
The class knows no architecture: it reads the spec.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import ops
from ..cache import SequenceCache
from ..config import ModelConfig, ModelSpec, load_config, resolve_dtype
from ..csrc import prepare
from ..parts import build_block, build_part
from ..weights import load_weights, random_state_on_device
from .step import StepContext, context_of, pack_step


def _walk(part):
    yield part
    for sub in part.sub_parts():
        yield from _walk(sub)


class Model:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device, attention: str = "auto"):
        spec.validate()
        self.spec = spec
        self.dtype = resolve_dtype(dtype)
        self.device = torch.device(device)
        self.attention = attention
        self.embedding = build_part("embedding", spec.embedding)
        self.blocks = [build_block(layer) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm)
        self.head = build_part("head", spec.head)
        self.err = None
        self.decode_scratch = None
        self.prefill_graphs = None  # engine.graphs.PrefillGraphs once enabled
        # a callable (index, hidden, delta) that is shown the float32 residual stream after the embedding (index 0) and
        # after every schedule entry (index k + 1); the stream's value there is hidden + delta when delta is pending.
        # For diagnosis (trace_run --dump-layers); it reads, it must not write.
        self.observer = None
        self._bound = False

    # ------------------------------------------------------------------ structure
    def parts(self):
        for top in (self.embedding, *self.blocks, self.final_norm, self.head):
            yield from _walk(top)

    def tensor_specs(self):
        return [t for part in self.parts() for t in part.tensor_specs()]

    @staticmethod
    def tensor_specs_of(spec: ModelSpec):
        """The tensors a model of this spec wants from its weight files (no device is touched)."""
        return Model(spec, torch.float32, "cpu").tensor_specs()

    def step_weight_bytes(self) -> int:
        """Bytes of weights that ONE step reads: every schedule entry's parts, the final norm and the head."""
        def of(top):
            return sum(t.numel() * t.element_size() for part in _walk(top) for t in part.step_weights())
        total = of(self.embedding) + of(self.final_norm) + of(self.head)
        return total + sum(of(self.blocks[entry.layer]) for entry in self.spec.schedule)

    def cache_needs(self) -> list:
        """Per schedule entry: what its mixer keeps per sequence; None when it reads another entry's cache."""
        return [None if e.cache_from is not None else self.blocks[e.layer].cache_need() for e in self.spec.schedule]

    # ------------------------------------------------------------------ weights
    def bind(self, tensors) -> "Model":
        ops.require_cuda(self.device, "the model")
        if self.device.type == "cuda" and self.device.index is not None:
            torch.cuda.set_device(self.device)  # the kernels launch on the current device's current stream
        libraries = {"embed", "norm"}
        for part in self.parts():
            libraries |= part.kernel_libraries(self.dtype)
        prepare(libraries)
        for part in self.parts():
            part.bind(tensors, self.dtype, self.device)
        self.err = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.decode_scratch = ops.DecodeScratch(self.device)
        self._bound = True
        return self

    @classmethod
    def from_dir(cls, model_dir, dtype="auto", device="cuda", attention: str = "auto") -> "Model":
        config = load_config(model_dir)
        return cls.from_config(config, model_dir, dtype, device, attention)

    @classmethod
    def from_config(cls, config: ModelConfig, model_dir, dtype="auto", device="cuda", attention: str = "auto") -> "Model":
        resolved = resolve_dtype(dtype, getattr(config, "torch_dtype", None))
        model = cls(config.model_spec(), resolved, device, attention)
        model.config = config
        tensors = load_weights(model_dir, model.tensor_specs(), resolved, model.device, model.spec.redundant_tensors)
        return model.bind(tensors)

    @classmethod
    def from_random(cls, config: ModelConfig, seed: int = 0, dtype="bfloat16", device="cuda", attention: str = "auto") -> "Model":
        """A model of `config` whose weights are drawn on the device (no model folder): for measurements at sizes of
        tens of GB. `write_random_model` + `from_dir` is the mode whose weights a plain implementation can read."""
        resolved = resolve_dtype(dtype, getattr(config, "torch_dtype", None))
        model = cls(config.model_spec(), resolved, device, attention)
        model.config = config
        ops.require_cuda(model.device, "the model")
        return model.bind(random_state_on_device(model.tensor_specs(), seed, resolved, model.device))

    # ------------------------------------------------------------------ cache
    def new_cache(self, max_tokens: int, max_seqs: int = 256, max_len: Optional[int] = None) -> SequenceCache:
        limit = self.spec.max_positions if max_len is None else min(max_len, self.spec.max_positions)
        return SequenceCache(self.cache_needs(), max_tokens, max_seqs, limit, self.dtype, self.device)

    # ------------------------------------------------------------------ the step
    def forward(self, ctx: StepContext, cache: SequenceCache) -> Optional[torch.Tensor]:
        """Run the schedule over the context's tokens; logits of ctx.want_rows (None if nothing is wanted)."""
        ctx.step_memo = {}
        hidden = ctx.embedded if ctx.embedded is not None else self.embedding.forward(ctx.token_ids, ctx)
        delta = None
        if self.observer is not None:
            self.observer(0, hidden, None)
        for index, entry in enumerate(self.spec.schedule):
            own = entry.cache_from is None
            site = cache.site(index if own else entry.cache_from)
            delta = self.blocks[entry.layer].forward(hidden, delta, ctx, site, own)
            if self.observer is not None:
                self.observer(index + 1, hidden, delta)
        if ctx.want_rows is None:
            return None
        shape = (ctx.want_rows.numel(), hidden.shape[1])
        rms = self.final_norm.fused_rms()
        if rms is not None and (delta is None or delta.dtype == rms[0].dtype):
            # the wanted rows are gathered and normalised by one kernel
            normed = torch.empty(shape, dtype=rms[0].dtype, device=hidden.device)
            ops.gather_rows_norm(hidden, delta, ctx.want_rows, rms[0], rms[1], normed, ctx.err)
            return self.head.forward(normed)
        rows = torch.empty(shape, dtype=torch.float32, device=hidden.device)
        ops.gather_rows(hidden, delta, ctx.want_rows, rows, ctx.err)
        return self.head.forward(self.final_norm.forward(rows, None))

    def step(self, cache: SequenceCache, entries: Sequence[tuple[int, Sequence[int]]],
             want: Optional[Sequence[Sequence[int]]] = None, extras: Optional[dict] = None) -> Optional[torch.Tensor]:
        """One step of a batch.

        entries  (slot, next token ids) per sequence; slot -1 is a padding entry. Each sequence's tokens
                 continue at its own length in the cache; its keys/values (or state) are appended.
        want     per entry the places among its tokens whose logits are wanted; None = each entry's last.
        extras   name -> per entry an array [tokens of the entry, ...]: side inputs for parts that read
                 `ctx.extras[name]` (say, positions on several axes); laid out like the tokens, [T, ...].
        Returns float32 logits [wanted, vocab] in the order of the entries and of `want`.
        """
        if not self._bound:
            raise RuntimeError("the model has no weights yet (bind() or from_dir())")
        if not entries:
            return None
        triples = []
        grow = []
        for slot, tokens in entries:
            start = cache.lengths[slot] if slot >= 0 else 0
            if slot >= 0:
                total = start + len(tokens)
                if total > self.spec.max_positions:
                    raise ValueError(f"Requested sequence length {total} exceeds model limit {self.spec.max_positions}")
                grow.append((slot, total))
            triples.append((slot, start, tokens))
        if len({s for s, _ in grow}) != len(grow):
            raise ValueError("step: a slot appears twice in one batch")
        cache.reserve(grow)
        cache.flush()
        step = pack_step(triples, want)
        logits, replayed = None, False
        if self.prefill_graphs is not None and not extras and self.prefill_graphs.takes(step):
            before = self.prefill_graphs.replays
            logits = self.prefill_graphs.run(cache, step, triples, want)
            replayed = self.prefill_graphs.replays > before
        if not replayed:
            # from pageable memory the copy is complete when the call returns, so the host array may go
            dev = torch.from_numpy(step.packed).to(self.device)
            ctx = context_of(step, dev, self.err, self.dtype, self.attention, self.decode_scratch)
            if extras:
                ctx.extras = {}
                for name, per_entry in extras.items():
                    pieces = [torch.as_tensor(piece) for piece in per_entry]
                    if [len(piece) for piece in pieces] != step.host_q_lens:
                        raise ValueError(f"step: extra input {name!r} does not have one row per token of every entry")
                    ctx.extras[name] = torch.cat(pieces).to(self.device)
            logits = self.forward(ctx, cache)
        for slot, tokens in entries:
            if slot >= 0:
                cache.advance(slot, len(tokens))
        return logits

    def enable_prefill_graphs(self, on: bool = True) -> None:
        """Replay steps of whole prompts whose shape comes back from CUDA graphs (bfloat16, graph-safe parts only)."""
        from .graphs import GraphDecoder, PrefillGraphs
        usable = on and self.dtype == torch.bfloat16 and self.device.type == "cuda" and GraphDecoder.supported(self)
        self.prefill_graphs = PrefillGraphs(self) if usable else None

    def raise_on_kernel_error(self) -> None:
        """Read the device error word (synchronises) and raise if a kernel met a bad index."""
        word = int(self.err.item())
        if word:
            self.err.zero_()
            raise ops.KernelError("kernel error: " + ops.describe_error_word(word))
