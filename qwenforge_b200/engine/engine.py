"""The Python entry point, in the reference's manner (student_engine.py:309-317, :1380-1399):

    engine = StudentEngine(model_path, device="cuda", dtype="bfloat16", attn_implementation="sdpa",
                           local_files_only=False, seed=0)
    texts  = engine.generate(prompts, max_new_tokens, batch_size=1, suite_name=None)

with the same names and meanings: `device` a torch device string (CUDA only here), `dtype` one of
auto / bfloat16 / bf16 / float32 / fp32, `attn_implementation` "sdpa" for the fastest attention kernels
that take the shapes and anything else for the plain SIMT kernel (the reference: "sdpa" or eager math,
:609, :645), `local_files_only` for the tokenizer, `seed` for sampling, `batch_size` the number of
prompts that start together, `suite_name` accepted and never read. `generate` returns one string per
prompt, `[]` for no prompts and `""` for a budget <= 0 (:1388-1394).

`generate_ids` is the same on token ids, with temperature, stop tokens and per-request budgets.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..cache import PAGE_TOKENS, CacheFull, round_up
from ..sampling import Sampler, SamplingParams
from ..weights.resolve import resolve_model_dir
from .generate import GenerationLoop, SequenceResult
from .graphs import MAX_STOP_IDS, GraphDecoder
from .model import Model
from .tokenizer import load_tokenizer


class ModelStepper:
    """The generation loop's view of a model, its cache and a sampler (`generate.Stepper`)."""

    def __init__(self, model: Model, cache, sampler: Sampler, graph_decoder: Optional[GraphDecoder] = None,
                 min_graph_steps: int = 8):
        self.model = model
        self.cache = cache
        self.sampler = sampler
        self.max_positions = model.spec.max_positions
        self.graph_decoder = graph_decoder
        self.min_graph_steps = min_graph_steps  # the reference graphs runs of >= 8 new tokens (student_engine.py:1274-1276)

    def open(self) -> int:
        return self.cache.open()

    def close(self, slot: int) -> None:
        self.cache.close(slot)

    def reserve(self, slot_totals) -> None:
        self.cache.reserve(list(slot_totals))

    def step_and_choose(self, entries, seq_ids, steps) -> list[int]:
        logits = self.model.step(self.cache, entries)
        device = logits.device
        ids = steps_t = None
        if not self.sampler.greedy:
            ids = torch.tensor(list(seq_ids), dtype=torch.int64).to(device)
            steps_t = torch.tensor(list(steps), dtype=torch.int32).to(device)
        chosen = self.sampler(logits, ids, steps_t)
        packed = torch.cat((chosen, self.model.err)).tolist()  # one copy back: the tokens and the error word
        if packed[-1]:
            self.model.raise_on_kernel_error()
        return packed[:-1]


    def open_decode_session(self, rows, stop_token_ids):
        """A CUDA-graph decode session for these rows, or None when graphs are off, a part of the model plans on the
        host, or the run is too short to repay a capture."""
        if self.graph_decoder is None or len(rows) > 1024 or len(stop_token_ids) > MAX_STOP_IDS:
            return None
        if max(budget - made for _, _, _, made, budget in rows) < self.min_graph_steps:
            return None
        return _GraphSession(self, rows, stop_token_ids)


class _GraphSession:
    def __init__(self, stepper: ModelStepper, rows, stop_token_ids):
        cache = stepper.cache
        self.stepper = stepper
        self.slots = [r[0] for r in rows]
        longest = max(cache.lengths[slot] + (budget - made) for slot, _, _, made, budget in rows)
        self.graph = stepper.graph_decoder.get(len(rows), longest, stepper.sampler)
        cache.flush()
        self.graph.load(self.slots, [r[1] for r in rows], [cache.lengths[r[0]] for r in rows], [r[3] for r in rows],
                        [r[4] for r in rows], [r[2] for r in rows], stop_token_ids)
        self.in_flight = 0   # steps already on the stream whose tokens have not been read

    def run(self, n_steps: int) -> list:
        """The next chunk's tokens, per step and row. The rows' state lives on the device, and a row that ends turns
        into a padding entry there by itself, so the chunk after this one goes onto the stream as soon as the device
        says that some row is still live, before the host has looked at a single token: the GPU works on it while the
        caller applies its decisions to this chunk."""
        n = self.in_flight or self.graph.enqueue(n_steps)
        produced, left, err = self.graph.collect(n)
        self.in_flight = self.graph.enqueue(left) if left > 0 else 0
        cache = self.stepper.cache
        for row, slot in enumerate(self.slots):
            fed = sum(1 for step_tokens in produced if step_tokens[row] >= 0)
            if fed:
                cache.advance(slot, fed)
        if err:
            self.stepper.model.raise_on_kernel_error()
        return [step_tokens[:len(self.slots)] for step_tokens in produced]


class StudentEngine:
    def __init__(self, model_path: str, device: str = "cuda", dtype: str = "bfloat16",
                 attn_implementation: str = "sdpa", local_files_only: bool = False, seed: int = 0,
                 max_cache_tokens: Optional[int] = None, cuda_graphs: bool = True):
        self.model_path = model_path
        self.device = torch.device(device)
        self.attn_implementation = str(attn_implementation).lower()
        self.local_files_only = bool(local_files_only)
        self.seed = int(seed)
        model_dir = resolve_model_dir(model_path)
        attention = "auto" if self.attn_implementation in ("sdpa", "flash", "auto") else "generic"
        self.model = Model.from_dir(model_dir, dtype, self.device, attention)
        self.config = self.model.config
        self.torch_dtype = self.model.dtype
        self.tokenizer = load_tokenizer(model_dir, self.model.spec.vocab_size, self.local_files_only)
        self._max_cache_tokens = max_cache_tokens
        self.cuda_graphs = bool(cuda_graphs) and self.device.type == "cuda" and GraphDecoder.supported(self.model)
        if self.cuda_graphs:
            self.model.enable_prefill_graphs()  # prompts whose shape comes back are replayed too
        self.cache = None
        self.graph_decoder: Optional[GraphDecoder] = None
        self.last_loop: Optional[GenerationLoop] = None

    # ------------------------------------------------------------------ cache sizing
    def _ensure_cache(self, prompt_lengths: Sequence[int], budgets: Sequence[int], batch_size: int) -> None:
        """A cache that holds the largest batch of this call; kept and reused while it is large enough."""
        need_tokens = need_seqs = 0
        for begin in range(0, len(prompt_lengths), batch_size):
            chunk = range(begin, min(begin + batch_size, len(prompt_lengths)))
            tokens = sum(round_up(max(prompt_lengths[i], 1) + max(budgets[i], 1), PAGE_TOKENS) for i in chunk)
            need_tokens, need_seqs = max(need_tokens, tokens), max(need_seqs, len(chunk))
        if self._max_cache_tokens is not None:
            if need_tokens > self._max_cache_tokens:
                raise CacheFull(f"a batch of this call needs {need_tokens} cache tokens; "
                                f"max_cache_tokens is {self._max_cache_tokens}")
            need_tokens = self._max_cache_tokens
        cache = self.cache
        if cache is None or cache.n_pages * PAGE_TOKENS < need_tokens or cache.max_seqs < need_seqs:
            if cache is not None and cache.live_slots():
                raise RuntimeError("the cache cannot grow while sequences are live")
            self.cache = self.graph_decoder = None  # graphs hold the old cache's addresses
            del cache
            self.cache = self.model.new_cache(need_tokens, max(need_seqs, 8))
        if self.cuda_graphs and self.graph_decoder is None:
            self.graph_decoder = GraphDecoder(self.model, self.cache)

    # ------------------------------------------------------------------ token ids
    @torch.inference_mode()
    def generate_ids(self, prompts: Sequence[Sequence[int]], max_new_tokens, batch_size: int = 1,
                     temperature: float = 0.0, seed: Optional[int] = None,
                     stop_token_ids: Optional[Sequence[int]] = None, ignore_eos: bool = False) -> list[list[int]]:
        return [r.tokens for r in self.generate_results(prompts, max_new_tokens, batch_size, temperature, seed,
                                                        stop_token_ids, ignore_eos)]

    @torch.inference_mode()
    def generate_results(self, prompts, max_new_tokens, batch_size: int = 1, temperature: float = 0.0,
                         seed: Optional[int] = None, stop_token_ids: Optional[Sequence[int]] = None,
                         ignore_eos: bool = False) -> list[SequenceResult]:
        prompts = [list(p) for p in prompts]
        if not prompts:
            return []
        n = len(prompts)
        budgets = [int(max_new_tokens)] * n if isinstance(max_new_tokens, int) else [int(b) for b in max_new_tokens]
        size = max(int(batch_size), 1)
        stops = self.model.spec.stop_token_ids if stop_token_ids is None else tuple(stop_token_ids)
        self._ensure_cache([len(p) for p in prompts], budgets, size)
        sampler = Sampler(SamplingParams(float(temperature), self.seed if seed is None else int(seed)))
        loop = GenerationLoop(ModelStepper(self.model, self.cache, sampler, self.graph_decoder), stops, ignore_eos,
                              getattr(self.tokenizer, "bos_token_id", None))
        self.last_loop = loop
        return loop.run(prompts, budgets, size)

    # ------------------------------------------------------------------ strings
    @torch.inference_mode()
    def generate(self, prompts: list, max_new_tokens: int, batch_size: int = 1, suite_name: Optional[str] = None) -> list:
        if not isinstance(prompts, list) or not all(isinstance(item, str) for item in prompts):
            raise TypeError("prompts must be list[str]")
        if not prompts:
            return []
        budget = int(max_new_tokens)
        if budget <= 0:
            return ["" for _ in prompts]
        ids = [self.tokenizer.encode_prompt(p) for p in prompts]
        # the reference generates exactly `max_new_tokens` tokens and ignores end-of-sequence tokens
        out = self.generate_ids(ids, budget, batch_size, ignore_eos=True)
        return [self.tokenizer.decode(tokens) for tokens in out]
