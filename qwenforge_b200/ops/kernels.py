"""Python entry of every CUDA kernel: argument checks, pointer passing, error codes.

Each function checks dtypes, shapes and contiguity on the host, then calls the exported C
function of its library with raw device pointers and the current stream. There is no other
implementation behind these names: tensors that are not on a CUDA device are refused, and a
missing or failing kernel library raises `KernelLibraryError`.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..csrc import library

_P = ctypes.c_void_p
_I = ctypes.c_int
_LL = ctypes.c_longlong
_ULL = ctypes.c_ulonglong
_F = ctypes.c_float

ERR_TOKEN_RANGE = 1
ERR_NO_PAGE = 2
ERR_ROW_RANGE = 4
ERR_COPY_TIMEOUT = 8
ERR_BARRIER_TIMEOUT = 16

_ERROR_TEXT = {
    ERR_TOKEN_RANGE: "a token id lies outside the embedding table",
    ERR_NO_PAGE: "a position was read or written whose cache page is not held by its sequence",
    ERR_ROW_RANGE: "a wanted row lies outside the step's tokens",
    ERR_COPY_TIMEOUT: "a bulk copy into shared memory did not complete within its wait limit",
    ERR_BARRIER_TIMEOUT: "the blocks of a persistent kernel did not all reach a barrier within its wait limit",
}


class KernelError(RuntimeError):
    pass


def describe_error_word(word: int) -> str:
    return "; ".join(text for bit, text in _ERROR_TEXT.items() if word & bit) or f"unknown error word {word}"


def require_cuda(device, what: str = "this operation") -> None:
    """There is no CPU execution path: anything that is to compute must live on a CUDA device."""
    if torch.device(device).type != "cuda":
        raise KernelError(f"{what} is on {device}: this library computes on CUDA devices only "
                          "(there is no CPU execution path)")
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device is available; this library has no CPU execution path")


launches = 0  # kernels of this library launched by this process (the measurement reads it)

_sm_counts: dict = {}


def sm_count(device) -> int:
    """Streaming multiprocessors of `device` (asked once): what grids and split counts are sized by."""
    device = torch.device(device)
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _sm_counts:
        _sm_counts[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return _sm_counts[index]


def _check(code: int, what: str) -> None:
    global launches
    launches += 1
    if code != 0:
        raise KernelError(f"{what}: CUDA error {code} at launch")


def _stream() -> _P:
    """The current stream's raw handle on the current device (the short way: this runs once per kernel launch)."""
    return _P(torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice()))


def _ptr(t: Optional[torch.Tensor]) -> _P:
    return _P(0) if t is None else _P(t.data_ptr())


def _dev(name: str, t: torch.Tensor, dtype=None, contiguous: bool = True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} is on {t.device}: the kernels of this library run on CUDA devices only")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} has dtype {t.dtype}, expected {dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} is not contiguous")


def _is_bf16(dtype: torch.dtype) -> int:
    if dtype == torch.bfloat16:
        return 1
    if dtype == torch.float32:
        return 0
    raise KernelError(f"activation dtype {dtype} is not supported (bfloat16 or float32)")


class KvSiteArgs:
    """What the kernels need to address one schedule entry's keys and values (see `cache.KvSite`)."""
    __slots__ = ("storage", "table", "page_elems", "table_stride", "kv_heads", "head_dim")

    def __init__(self, storage: torch.Tensor, table: torch.Tensor, kv_heads: int, head_dim: int):
        # storage: [pages, 2, kv_heads, PAGE, head_dim]; table: [slots, max_pages] int32
        self.storage = storage
        self.table = table
        self.page_elems = storage.stride(0)
        self.table_stride = table.stride(0)
        self.kv_heads = kv_heads
        self.head_dim = head_dim


def embed_gather(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, err: torch.Tensor) -> None:
    """out[t] = float32(table[ids[t]]); ids int32 [T], table [V, W], out float32 [T, W]."""
    _dev("ids", ids, torch.int32)
    _dev("table", table)
    _dev("out", out, torch.float32)
    n, (vocab, width) = ids.numel(), table.shape
    if out.shape != (n, width):
        raise KernelError(f"embed_gather: out is {tuple(out.shape)}, expected {(n, width)}")
    _check(library("embed").qf_embed_gather(_I(_is_bf16(table.dtype)), _ptr(ids), _ptr(table), _ptr(out), _I(n),
                                            _I(vocab), _I(width), _ptr(err), _stream()), "embed_gather")


def gather_rows(hidden: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor, out: torch.Tensor,
                err: torch.Tensor) -> None:
    """out[r] = hidden[rows[r]] + delta[rows[r]] in float32; delta may be None."""
    _dev("hidden", hidden, torch.float32)
    _dev("rows", rows, torch.int32)
    _dev("out", out, torch.float32)
    n_in, width = hidden.shape
    is_bf16 = 0
    if delta is not None:
        _dev("delta", delta)
        is_bf16 = _is_bf16(delta.dtype)
        if delta.shape != hidden.shape:
            raise KernelError("gather_rows: delta and hidden differ in shape")
    if out.shape != (rows.numel(), width):
        raise KernelError("gather_rows: out has the wrong shape")
    _check(library("embed").qf_gather_rows(_I(is_bf16), _ptr(hidden), _ptr(delta), _ptr(rows), _ptr(out),
                                           _I(rows.numel()), _I(n_in), _I(width), _ptr(err), _stream()), "gather_rows")


def gather_rows_norm(hidden: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor, weight: torch.Tensor,
                     eps: float, out: torch.Tensor, err: torch.Tensor) -> None:
    """out[r] = rmsnorm(hidden[rows[r]] + delta[rows[r]]) * weight, the sums in float32; delta may be None. hidden float32
    [T, W]; delta, weight and out share a dtype."""
    _dev("hidden", hidden, torch.float32)
    _dev("rows", rows, torch.int32)
    _dev("weight", weight)
    _dev("out", out, weight.dtype)
    n_in, width = hidden.shape
    if delta is not None:
        _dev("delta", delta, weight.dtype)
        if delta.shape != hidden.shape:
            raise KernelError("gather_rows_norm: delta and hidden differ in shape")
    if out.shape != (rows.numel(), width) or weight.numel() != width:
        raise KernelError("gather_rows_norm: out must be [rows, width], weight [width]")
    _check(library("embed").qf_gather_rows_norm(_I(_is_bf16(weight.dtype)), _ptr(hidden), _ptr(delta), _ptr(rows),
                                                _ptr(weight), _ptr(out), _I(rows.numel()), _I(n_in), _I(width), _F(eps),
                                                _ptr(err), _stream()), "gather_rows_norm")


def add_rms_norm(hidden: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                 out: torch.Tensor) -> None:
    """hidden += delta (if given); out = rmsnorm(hidden) * weight. hidden float32 [R, W]; out, weight, delta share a dtype."""
    _dev("hidden", hidden, torch.float32)
    _dev("weight", weight)
    _dev("out", out, weight.dtype)
    rows, width = hidden.shape
    if weight.shape != (width,) or out.shape != hidden.shape:
        raise KernelError("add_rms_norm: shapes of weight/out do not match hidden")
    if delta is not None:
        _dev("delta", delta, weight.dtype)
        if delta.shape != hidden.shape:
            raise KernelError("add_rms_norm: delta and hidden differ in shape")
    _check(library("norm").qf_add_rms_norm(_I(_is_bf16(weight.dtype)), _ptr(hidden), _ptr(delta), _ptr(weight),
                                           _ptr(out), _I(rows), _I(width), _F(eps), _stream()), "add_rms_norm")


def gemm_f32(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out = x @ weight.T (+ bias) in true float32 (FFMA; no TF32). x [M, K], weight [N, K], out [M, N]; rows may be strided."""
    for name, t in (("x", x), ("weight", weight), ("out", out)):
        _dev(name, t, torch.float32, contiguous=False)
        if t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"gemm_f32: {name} must be 2-d with unit inner stride")
    (m, k), (n, k2) = x.shape, weight.shape
    if k != k2 or out.shape != (m, n):
        raise KernelError(f"gemm_f32: shapes {tuple(x.shape)} x {tuple(weight.shape)}^T -> {tuple(out.shape)} do not agree")
    if bias is not None:
        _dev("bias", bias, torch.float32)
        if bias.shape != (n,):
            raise KernelError("gemm_f32: bias has the wrong shape")
    _check(library("gemm_f32").qf_gemm_f32(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), _I(m), _I(n), _I(k),
                                           _I(x.stride(0)), _I(weight.stride(0)), _I(out.stride(0)), _stream()),
           "gemm_f32")


def rope_cache_write(qkv: torch.Tensor, tok_seq: torch.Tensor, tok_pos: torch.Tensor, slots: torch.Tensor,
                     inv_freq: Optional[torch.Tensor], rot_dim: int, n_heads: int, q_out: torch.Tensor,
                     site: KvSiteArgs, write_cache: bool, err: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
    """Rotate q and k heads of qkv [T, (NH + 2 KVH) D] by position, write q to q_out [T, NH D] and k, v into the cache."""
    _dev("qkv", qkv)
    _dev("q_out", q_out, qkv.dtype)
    _dev("cache", site.storage, qkv.dtype)
    _dev("tok_seq", tok_seq, torch.int32)
    _dev("tok_pos", tok_pos, torch.int32)
    _dev("slots", slots, torch.int32)
    n = qkv.shape[0]
    d, kvh = site.head_dim, site.kv_heads
    if qkv.shape[1] != (n_heads + 2 * kvh) * d or q_out.shape != (n, n_heads * d):
        raise KernelError("rope_cache_write: qkv/q_out widths do not match the head counts")
    if bias is not None:
        _dev("bias", bias, qkv.dtype)
        if bias.numel() != qkv.shape[1]:
            raise KernelError("rope_cache_write: bias must have one element per projection column")
    if inv_freq is not None:
        _dev("inv_freq", inv_freq, torch.float32)
        if inv_freq.numel() * 2 != rot_dim:
            raise KernelError("rope_cache_write: inv_freq must hold rot_dim / 2 frequencies")
    _check(library("rope_cache").qf_rope_cache_write(
        _I(_is_bf16(qkv.dtype)), _ptr(qkv), _ptr(bias), _I(qkv.stride(0)), _ptr(tok_seq), _ptr(tok_pos), _ptr(slots),
        _ptr(inv_freq), _I(rot_dim), _I(n_heads), _ptr(q_out), _ptr(site.storage), _ptr(site.table),
        _LL(site.page_elems), _I(site.table_stride), _I(kvh), _I(d), _I(1 if write_cache else 0), _I(n), _ptr(err),
        _stream()), "rope_cache_write")


GENERIC_DECODE_CHUNK = 256


def attention_generic(q: torch.Tensor, out: torch.Tensor, cu_q: torch.Tensor, tok_pos: torch.Tensor,
                      slots: torch.Tensor, site: KvSiteArgs, n_heads: int, n_seqs: int, max_q_len: int, scale: float,
                      window: int, err: torch.Tensor, scratch: Optional["DecodeScratch"] = None,
                      max_kv_len: Optional[int] = None) -> None:
    """Causal grouped-query attention of the step's queries over each sequence's cache (any sizes, SIMT float32 math).
    A step of one token per sequence whose longest sequence exceeds one chunk of 256 keys is cut into chunks of keys
    when `scratch` and `max_kv_len` (a bound on any sequence's length after the step) are given: a block per chunk,
    then a fold in rising order; which chunks a row has depends on its own position only."""
    _dev("q", q)
    _dev("out", out, q.dtype)
    _dev("cache", site.storage, q.dtype)
    d = site.head_dim
    if d > 256:
        raise KernelError(f"attention_generic: head_dim {d} > 256 is not supported")
    if q.shape[1] != n_heads * d or out.shape != q.shape:
        raise KernelError("attention_generic: q/out widths do not match the head count")
    if (scratch is not None and max_kv_len is not None and max_q_len == 1 and q.shape[0] == n_seqs
            and max_kv_len > GENERIC_DECODE_CHUNK):
        n_chunks = -(-int(max_kv_len) // GENERIC_DECODE_CHUNK)
        scratch.ensure(n_seqs, n_heads, n_chunks, d, 0)
        _check(library("attention_generic").qf_attention_generic_decode(
            _I(_is_bf16(q.dtype)), _ptr(q), _ptr(out), _ptr(cu_q), _ptr(tok_pos), _ptr(slots), _ptr(site.storage),
            _ptr(site.table), _LL(site.page_elems), _I(site.table_stride), _I(site.kv_heads), _I(d), _I(n_heads),
            _I(n_seqs), _I(int(max_kv_len)), _F(scale), _I(window), _ptr(scratch.part_o), _ptr(scratch.part_ml), _ptr(err),
            _stream()), "attention_generic")
        return
    _check(library("attention_generic").qf_attention_generic(
        _I(_is_bf16(q.dtype)), _ptr(q), _ptr(out), _ptr(cu_q), _ptr(tok_pos), _ptr(slots), _ptr(site.storage),
        _ptr(site.table), _LL(site.page_elems), _I(site.table_stride), _I(site.kv_heads), _I(d), _I(n_heads),
        _I(n_seqs), _I(max_q_len), _F(scale), _I(window), _ptr(err), _stream()), "attention_generic")


FAST_ATTENTION_HEAD_DIMS = (32, 64, 96, 128)


def attention_prefill(q: torch.Tensor, out: torch.Tensor, cu_q: torch.Tensor, tok_pos: torch.Tensor,
                      slots: torch.Tensor, site: KvSiteArgs, n_heads: int, n_seqs: int, max_q_len: int, scale: float,
                      window: int, err: torch.Tensor, max_kv_len: Optional[int] = None) -> None:
    """Tensor-core flash attention of spans of new tokens over the cache: bfloat16, head sizes 32/64/96/128.
    `max_kv_len`: an upper bound of any sequence's length after the step (None: unknown, taken as long); it only
    steers whether a tile of rows shares its pages among two groups of warps."""
    _dev("q", q, torch.bfloat16)
    _dev("out", out, torch.bfloat16)
    _dev("cache", site.storage, torch.bfloat16)
    d = site.head_dim
    if d not in FAST_ATTENTION_HEAD_DIMS:
        raise KernelError(f"attention_prefill: head_dim {d} has no tensor-core kernel (have {FAST_ATTENTION_HEAD_DIMS}); "
                          "use attention_generic")
    if q.shape[1] != n_heads * d or out.shape != q.shape:
        raise KernelError("attention_prefill: q/out widths do not match the head count")
    _check(library("attention_prefill").qf_attention_prefill(
        _ptr(q), _ptr(out), _ptr(cu_q), _ptr(tok_pos), _ptr(slots), _ptr(site.storage), _ptr(site.table),
        _LL(site.page_elems), _I(site.table_stride), _I(site.kv_heads), _I(d), _I(n_heads), _I(n_seqs), _I(q.shape[0]),
        _I(max_q_len), _I(1 << 30 if max_kv_len is None else int(max_kv_len)), _F(scale), _I(window), _ptr(err), _stream()),
        "attention_prefill")


TC_ATTENTION_HEAD_DIMS = (64, 128)


def attention_prefill_tc(q: torch.Tensor, out: torch.Tensor, cu_q: torch.Tensor, tok_pos: torch.Tensor,
                         slots: torch.Tensor, site: KvSiteArgs, n_heads: int, n_seqs: int, max_q_len: int, scale: float,
                         window: int, err: torch.Tensor, max_kv_len: Optional[int] = None) -> None:
    """The same attention on the fifth-generation tensor cores (tcgen05, accumulators in tensor memory): blocks of
    128 query rows; bfloat16, head sizes 64 and 128, cache pages without gaps. `max_kv_len` as in `attention_prefill`:
    with few tiles of many pages, two blocks of a cluster share a tile."""
    _dev("q", q, torch.bfloat16)
    _dev("out", out, torch.bfloat16)
    _dev("cache", site.storage, torch.bfloat16)
    d = site.head_dim
    if d not in TC_ATTENTION_HEAD_DIMS:
        raise KernelError(f"attention_prefill_tc: head_dim {d} has no tcgen05 kernel (have {TC_ATTENTION_HEAD_DIMS}); "
                          "use attention_prefill")
    if q.shape[1] != n_heads * d or out.shape != q.shape:
        raise KernelError("attention_prefill_tc: q/out widths do not match the head count")
    if site.page_elems != 2 * site.kv_heads * site.storage.shape[-2] * d:
        raise KernelError("attention_prefill_tc: the cache pages have gaps; use attention_prefill")
    _check(library("attention_prefill_tc").qf_attention_prefill_tc(
        _ptr(q), _ptr(out), _ptr(cu_q), _ptr(tok_pos), _ptr(slots), _ptr(site.storage), _ptr(site.table),
        _LL(site.page_elems), _I(site.table_stride), _I(site.kv_heads), _I(d), _I(n_heads), _I(n_seqs), _I(q.shape[0]),
        _I(max_q_len), _I(1 << 30 if max_kv_len is None else int(max_kv_len)), _F(scale), _I(window), _ptr(err), _stream()),
        "attention_prefill_tc")


class DecodeScratch:
    """Scratch of the split-K decode attention: float32 partial numerators and (max, sum) pairs per
    (sequence, head, split), and the ticket counters (kept zero between calls by the kernel itself).
    One instance is shared by all layers of a model: they run one after another on one stream."""

    def __init__(self, device):
        self.device = device
        self.part_o = self.part_ml = self.counters = None
        self.plans: dict = {}   # attention shape -> int32 [records, 4]: which block takes which run of which sequence

    def plan(self, key: tuple, records: int) -> torch.Tensor:
        held = self.plans.get(key)
        if held is None or held.shape[0] < records:
            held = self.plans[key] = torch.empty((records, 4), dtype=torch.int32, device=self.device)
        return held

    def ensure(self, n_seqs: int, n_heads: int, n_splits: int, head_dim: int, n_counters: int) -> None:
        rows = n_seqs * n_heads * n_splits
        if self.part_o is None or self.part_o.numel() < rows * head_dim:
            self.part_o = torch.empty(rows * head_dim, dtype=torch.float32, device=self.device)
        if self.part_ml is None or self.part_ml.numel() < rows * 2:
            self.part_ml = torch.empty(rows * 2, dtype=torch.float32, device=self.device)
        if n_counters and (self.counters is None or self.counters.numel() < n_counters):
            self.counters = torch.zeros(n_counters, dtype=torch.int32, device=self.device)


def attention_decode_warps(head_dim: int) -> int:
    """Warps of a block of the decode attention at this head size (each takes one page at a time): the fewest pages
    that a run of a sequence should hold."""
    return int(library("attention_decode").qf_attention_decode_warps(_I(head_dim)))


def attention_decode_plan(cu_q: torch.Tensor, tok_pos: torch.Tensor, slots: torch.Tensor, kv_heads: int, head_dim: int,
                          n_heads: int, n_seqs: int, window: int, n_splits: int, scratch: DecodeScratch) -> torch.Tensor:
    """The plan of one decode step for attention of this shape: which block takes which run of which sequence, worked
    out on the device from the batch's lengths (sequences of unequal lengths get blocks of about equal work; a batch
    that fills the SMs unsplit stays unsplit). One plan serves every layer of the step with this shape. `n_splits` is
    the most runs one sequence may get. The tensor belongs to `scratch` and is overwritten by the next plan of the
    same shape."""
    for name, t in (("cu_q", cu_q), ("tok_pos", tok_pos), ("slots", slots)):
        _dev(name, t, torch.int32)
    if not 1 <= n_splits <= 128:
        raise KernelError(f"attention_decode: n_splits {n_splits} outside 1..128")
    if kv_heads <= 0 or n_heads % kv_heads:
        raise KernelError(f"attention_decode: {n_heads} heads do not divide into {kv_heads} groups")
    lib = library("attention_decode")
    lib.qf_attention_decode_plan_size.restype = ctypes.c_longlong
    records = int(lib.qf_attention_decode_plan_size(_I(n_seqs), _I(kv_heads), _I(n_heads), _I(head_dim), _I(n_splits)))
    if records <= 0:
        raise KernelError(f"attention_decode: head_dim {head_dim} has no tensor-core kernel (have {FAST_ATTENTION_HEAD_DIMS})")
    plan = scratch.plan((n_seqs, kv_heads, n_heads, head_dim, window, n_splits), records)
    _check(lib.qf_attention_decode_plan(_ptr(cu_q), _ptr(tok_pos), _ptr(slots), _I(n_seqs), _I(kv_heads), _I(head_dim),
                                        _I(n_heads), _I(window), _I(n_splits), _ptr(plan), _stream()), "attention_decode_plan")
    return plan


def attention_decode(q: torch.Tensor, out: torch.Tensor, cu_q: torch.Tensor, tok_pos: torch.Tensor,
                     slots: torch.Tensor, site: KvSiteArgs, n_heads: int, n_seqs: int, scale: float, window: int,
                     n_splits: int, scratch: DecodeScratch, err: torch.Tensor, plan: Optional[torch.Tensor] = None,
                     fold_later: bool = False) -> None:
    """Split-K flash decoding: ONE new token per sequence over its cache; bfloat16, head sizes 32/64/96/128.
    `n_splits` is the most blocks that share one (sequence, kv head); `plan` (attention_decode_plan with the same
    shape, made in this step; made here when absent) says how many of them each sequence gets. With `fold_later` the
    kernel stops at the runs' partial results in `scratch` and writes no `out` (which may be None): `fold_project`
    folds them on its way into the output projection."""
    _dev("q", q, torch.bfloat16)
    if not fold_later:
        _dev("out", out, torch.bfloat16)
    _dev("cache", site.storage, torch.bfloat16)
    d = site.head_dim
    if d not in FAST_ATTENTION_HEAD_DIMS:
        raise KernelError(f"attention_decode: head_dim {d} has no tensor-core kernel (have {FAST_ATTENTION_HEAD_DIMS}); "
                          "use attention_generic")
    if q.shape != (n_seqs, n_heads * d) or (not fold_later and out.shape != q.shape):
        raise KernelError("attention_decode: wants exactly one token per sequence, q [n_seqs, n_heads * head_dim]")
    if not 1 <= n_splits <= 128:
        raise KernelError(f"attention_decode: n_splits {n_splits} outside 1..128")
    if plan is None:
        plan = attention_decode_plan(cu_q, tok_pos, slots, site.kv_heads, d, n_heads, n_seqs, window, n_splits, scratch)
    group = n_heads // site.kv_heads
    n_counters = n_seqs * site.kv_heads * ((group + 15) // 16)
    partials = n_splits > 1 or fold_later
    if partials:
        scratch.ensure(n_seqs, n_heads, n_splits, d, n_counters)
    _check(library("attention_decode").qf_attention_decode(
        _ptr(q), _ptr(None if fold_later else out), _ptr(cu_q), _ptr(plan), _ptr(site.storage), _ptr(site.table),
        _LL(site.page_elems), _I(site.table_stride), _I(site.kv_heads), _I(d), _I(n_heads), _I(n_seqs), _F(scale),
        _I(window), _I(n_splits), _I(1 if fold_later else 0), _ptr(scratch.part_o if partials else None),
        _ptr(scratch.part_ml if partials else None), _ptr(scratch.counters if partials else None), _ptr(err),
        _stream()), "attention_decode")


class _FoldProjectArgs(ctypes.Structure):
    _fields_ = [("part_o", _P), ("part_ml", _P), ("runs", _P), ("w", _P), ("hidden", _P), ("rows", _I), ("n", _I),
                ("ldw", _I), ("n_heads", _I), ("head_dim", _I), ("max_splits", _I)]


def fold_project_takes(rows: int, weight: torch.Tensor, hidden: torch.Tensor, n_heads: int, head_dim: int) -> bool:
    """Whether `fold_project` takes the output projection `weight` [N, n_heads * head_dim] for a step of `rows` rows."""
    if weight.dtype != torch.bfloat16 or hidden.dtype != torch.float32 or weight.dim() != 2 or weight.stride(1) != 1:
        return False
    if weight.shape[1] != n_heads * head_dim or not hidden.is_contiguous() or hidden.shape != (rows, weight.shape[0]):
        return False
    return bool(library("fold_project").qf_fold_project_takes(
        _I(rows), _I(weight.shape[0]), _I(weight.stride(0)), _I(n_heads), _I(head_dim), _ptr(weight), _ptr(hidden)))


FOLD_PROJECT_MAX_REDUCTIONS = 150_000


def fold_project_pays(rows: int, weight: torch.Tensor) -> bool:
    """Whether `fold_project` is the faster way for this projection. What it saves is the attention kernel's life after
    its pages (about 3 microseconds); what it costs grows with the 16-byte reductions into the stream, rows x N / 4 from
    each of its K / 32 blocks. Measured: 50,000 of them (8 rows, 896 x 896) gain 2.2 microseconds per layer, 524,000 (16
    rows, 2048 x 2048) lose 1."""
    return rows * weight.shape[0] * (weight.shape[1] // 32) // 4 <= FOLD_PROJECT_MAX_REDUCTIONS


def fold_project(plan: torch.Tensor, scratch: DecodeScratch, weight: torch.Tensor, hidden: torch.Tensor, n_heads: int,
                 head_dim: int, n_splits: int) -> None:
    """hidden[r, :] += fold(the partial results of sequence r) @ weight^T, after `attention_decode(..., fold_later=True)`
    with the same `plan`, `scratch` and `n_splits` in a step whose row r is sequence r (one token per sequence).
    bfloat16 weight [N, n_heads * head_dim], float32 hidden [rows, N]; the blocks' shares are added with atomic
    reductions, in no fixed order."""
    _dev("weight", weight, torch.bfloat16, contiguous=False)
    _dev("hidden", hidden, torch.float32)
    rows = hidden.shape[0]
    if not fold_project_takes(rows, weight, hidden, n_heads, head_dim):
        raise KernelError(f"fold_project: does not take {rows} rows, weight {tuple(weight.shape)}, {n_heads} heads of {head_dim}")
    if scratch.part_o is None or scratch.part_o.numel() < rows * n_heads * n_splits * head_dim:
        raise KernelError("fold_project: the scratch does not hold this step's partial results")
    a = _FoldProjectArgs(scratch.part_o.data_ptr(), scratch.part_ml.data_ptr(), plan.data_ptr(), weight.data_ptr(),
                         hidden.data_ptr(), rows, weight.shape[0], weight.stride(0), n_heads, head_dim, n_splits)
    _check(library("fold_project").qf_fold_project(ctypes.byref(a), _stream()), "fold_project")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    _dev("gate_up", gate_up)
    _dev("out", out, gate_up.dtype)
    rows, two_i = gate_up.shape
    if two_i % 2 or out.shape != (rows, two_i // 2):
        raise KernelError("swiglu: out must be [rows, width / 2]")
    _check(library("activation").qf_swiglu(_I(_is_bf16(gate_up.dtype)), _ptr(gate_up), _ptr(out), _I(rows),
                                           _I(two_i // 2), _stream()), "swiglu")


class SampleScratch:
    """Scratch of the sampling kernel when several blocks share a row: each block's best (score, id) and the
    rows' ticket counters (kept zero between calls by the kernel itself)."""

    def __init__(self):
        self.part_v = self.part_i = self.counters = None

    def ensure(self, rows: int, chunks: int, device) -> None:
        if self.part_v is None or self.part_v.numel() < rows * chunks or self.part_v.device != device:
            self.part_v = torch.empty(rows * chunks, dtype=torch.float32, device=device)
            self.part_i = torch.empty(rows * chunks, dtype=torch.int32, device=device)
        if self.counters is None or self.counters.numel() < rows or self.counters.device != device:
            self.counters = torch.zeros(rows, dtype=torch.int32, device=device)


_sample_scratch = SampleScratch()


def sample(logits: torch.Tensor, temperature: float, seed: int, seq_ids: Optional[torch.Tensor],
           steps: Optional[torch.Tensor], out: torch.Tensor, scratch: Optional[SampleScratch] = None) -> None:
    """out[r] = argmax (temperature <= 0) or a Gumbel-max draw keyed by (seed, seq_ids[r], steps[r]).
    `scratch`: whoever captures the call into a CUDA graph passes a scratch of its own, which then lives as long
    as the graph; other callers share one that grows as needed."""
    _dev("logits", logits, torch.float32, contiguous=False)
    _dev("out", out, torch.int32)
    if logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be 2-d with unit inner stride")
    rows, vocab = logits.shape
    if out.numel() != rows:
        raise KernelError("sample: out must have one element per row")
    if temperature > 0:
        if seq_ids is None or steps is None:
            raise KernelError("sample: sampling needs seq_ids and steps")
        _dev("seq_ids", seq_ids, torch.int64)
        _dev("steps", steps, torch.int32)
        if seq_ids.numel() != rows or steps.numel() != rows:
            raise KernelError("sample: seq_ids and steps must have one element per row")
    # enough blocks to fill the GPU (eight per SM) when there are few rows, at least 2048 tokens of the vocabulary each
    chunks = max(1, min(-(-vocab // 2048), -(-8 * sm_count(logits.device) // rows), 64))
    scratch = scratch or _sample_scratch
    if chunks > 1:
        scratch.ensure(rows, chunks, logits.device)
    _check(library("sampling").qf_sample(_ptr(logits), _I(rows), _I(vocab), _LL(logits.stride(0)),
                                         _F(max(float(temperature), 0.0)), _ULL(seed & 0xFFFFFFFFFFFFFFFF),
                                         _ptr(seq_ids), _ptr(steps), _ptr(out), _I(chunks),
                                         _ptr(scratch.part_v if chunks > 1 else None),
                                         _ptr(scratch.part_i if chunks > 1 else None),
                                         _ptr(scratch.counters if chunks > 1 else None), _stream()), "sample")


def decode_advance(sampled: torch.Tensor, token_ids: torch.Tensor, tok_pos: torch.Tensor, slots: torch.Tensor,
                   steps: torch.Tensor, budgets: torch.Tensor, stop_ids: torch.Tensor, n_stop: int,
                   out_tokens: torch.Tensor, cursor: torch.Tensor) -> None:
    """Record each live row's sampled token in out_tokens[cursor], feed it back as the next input, advance
    position and step count, retire rows that stopped (slot := -1); cursor += 1. All int32, on the device."""
    for name, t in (("sampled", sampled), ("token_ids", token_ids), ("tok_pos", tok_pos), ("slots", slots),
                    ("steps", steps), ("budgets", budgets), ("stop_ids", stop_ids), ("out_tokens", out_tokens),
                    ("cursor", cursor)):
        _dev(name, t, torch.int32)
    n = token_ids.numel()
    if out_tokens.dim() != 2 or out_tokens.shape[1] != n or n_stop > stop_ids.numel():
        raise KernelError("decode_advance: out_tokens must be [max_steps, rows]; n_stop within stop_ids")
    _check(library("decode_state").qf_decode_advance(
        _ptr(sampled), _ptr(token_ids), _ptr(tok_pos), _ptr(slots), _ptr(steps), _ptr(budgets), _ptr(stop_ids),
        _I(n_stop), _ptr(out_tokens), _ptr(cursor), _I(out_tokens.shape[0]), _I(n), _stream()), "decode_advance")


def decode_advance_embed(sampled: torch.Tensor, token_ids: torch.Tensor, tok_pos: torch.Tensor, slots: torch.Tensor,
                         steps: torch.Tensor, budgets: torch.Tensor, stop_ids: torch.Tensor, n_stop: int,
                         out_tokens: torch.Tensor, cursor: torch.Tensor, table: torch.Tensor, hidden: torch.Tensor,
                         ticket: torch.Tensor, err: torch.Tensor) -> None:
    """`decode_advance`, and the next step's embedding with it: hidden[r] = float32(table[the row's next input token]).
    `ticket` is one int32 that is zero before the first call."""
    for name, t in (("sampled", sampled), ("token_ids", token_ids), ("tok_pos", tok_pos), ("slots", slots),
                    ("steps", steps), ("budgets", budgets), ("stop_ids", stop_ids), ("out_tokens", out_tokens),
                    ("cursor", cursor), ("ticket", ticket)):
        _dev(name, t, torch.int32)
    _dev("table", table)
    _dev("hidden", hidden, torch.float32)
    n = token_ids.numel()
    if out_tokens.dim() != 2 or out_tokens.shape[1] != n or n_stop > stop_ids.numel():
        raise KernelError("decode_advance_embed: out_tokens must be [max_steps, rows]; n_stop within stop_ids")
    if table.dim() != 2 or hidden.shape != (n, table.shape[1]):
        raise KernelError("decode_advance_embed: hidden must be [rows, width of the table]")
    _check(library("decode_state").qf_decode_advance_embed(
        _ptr(sampled), _ptr(token_ids), _ptr(tok_pos), _ptr(slots), _ptr(steps), _ptr(budgets), _ptr(stop_ids),
        _I(n_stop), _ptr(out_tokens), _ptr(cursor), _I(out_tokens.shape[0]), _I(n), _I(_is_bf16(table.dtype)),
        _ptr(table), _I(table.shape[0]), _I(table.shape[1]), _ptr(hidden), _ptr(ticket), _ptr(err), _stream()),
        "decode_advance_embed")


# ---------------------------------------------------------------------------------------------- fused skinny products

SKINNY_MAX_ROWS = 16
EPI_PLAIN, EPI_RESIDUAL, EPI_SWIGLU, EPI_QKV = 0, 1, 2, 3


class _SkinnyArgs(ctypes.Structure):
    _fields_ = [
        ("w", _P), ("bias", _P), ("n", _I), ("k", _I), ("ldw", _I), ("m", _I),
        ("x", _P), ("ldx", _I), ("hidden", _P), ("norm_w", _P), ("eps", _F),
        ("out", _P), ("ldo", _I), ("out_f32", _I), ("residual", _P), ("inter", _I),
        ("n_heads", _I), ("kv_heads", _I), ("head_dim", _I), ("rot_dim", _I), ("write_cache", _I),
        ("inv_freq", _P), ("tok_pos", _P), ("tok_seq", _P), ("slots", _P), ("q_out", _P), ("kv_base", _P),
        ("table", _P), ("page_elems", _LL), ("table_stride", _I), ("err", _P),
    ]


_own_err_words = {}


def _err_word_for(device) -> torch.Tensor:
    """A device error word for calls that bring none of their own (kernel tests)."""
    key = str(device)
    if key not in _own_err_words:
        _own_err_words[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _own_err_words[key]


_skinny_answers: dict = {}


def skinny_gemm_takes(m: int, weight: torch.Tensor, epilogue: int = EPI_PLAIN, norm: bool = False, *,
                      ldx: Optional[int] = None, n_heads: int = 0, kv_heads: int = 0, head_dim: int = 0,
                      rot_dim: int = 0) -> bool:
    """Whether `skinny_gemm` runs `m` token rows against `weight` [N, K] with this epilogue and prologue. The answer
    is the library's own (`qf_skinny_gemm_takes` runs the planning of the launch without launching), so a shape
    that gets a yes here is never refused later. `ldx`: elements between input rows (default K); `rot_dim`: > 0 when
    the QKV epilogue is to rotate that many components of each head."""
    if not (weight.is_cuda and weight.dtype == torch.bfloat16 and weight.dim() == 2 and weight.stride(1) == 1):
        return False
    n, k = weight.shape
    key = (weight.device.index, int(m), n, k, weight.stride(0), epilogue, bool(norm), k if ldx is None else ldx,
           n_heads, kv_heads, head_dim, rot_dim)
    answer = _skinny_answers.get(key)
    if answer is None:
        with torch.cuda.device(weight.device):
            answer = library("skinny_gemm").qf_skinny_gemm_takes(
                _I(epilogue), _I(int(bool(norm))), _I(int(m)), _I(n), _I(k), _I(weight.stride(0)), _I(key[7]),
                _I(n // 2 if epilogue == EPI_SWIGLU else 0), _I(n_heads), _I(kv_heads), _I(head_dim),
                _I(1 if rot_dim > 0 else 0), _I(rot_dim)) != 0
        _skinny_answers[key] = answer
    return answer


def skinny_gemm_pays(m: int, weight: torch.Tensor) -> bool:
    """Whether the weight-streaming kernel is the faster way to run `m` token rows against `weight`, by measurement on
    a B200 (`python -m qwenforge_b200.measure products`): for weights of 100 MB and more it loses to the norm kernel,
    the library product and the elementwise kernel together (Qwen2.5-7B's feed-forward, 272 and 136 MB: 57 and 41
    microseconds against 52 and 30 at 8 rows, 62 and 51 against 52 and 31 at 16), and from 9 rows on already for
    weights above 64 MB (Qwen2.5-3B's gate/up, 90 MB: 24.4 against 22.3). Everything smaller it wins, the smaller the
    clearer (0.5B at 8 rows: 2.9 / 5.9 / 4.8 / 4.4 microseconds against 5.1 / 8.6 / 11.0 / 8.3)."""
    size = weight.numel() * weight.element_size()
    return size < 100e6 and (m <= 8 or size < 64e6)


def _skinny_args(epilogue: int, weight: torch.Tensor, *, x: Optional[torch.Tensor] = None,
                 hidden: Optional[torch.Tensor] = None, norm_weight: Optional[torch.Tensor] = None, eps: float = 0.0,
                 bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                 residual: Optional[torch.Tensor] = None, qkv: Optional[dict] = None,
                 err: Optional[torch.Tensor] = None):
    """Checks one fused product's tensors and fills the kernels' argument block; returns (block, norm flag)."""
    _dev("weight", weight, torch.bfloat16, contiguous=False)
    a = _SkinnyArgs()
    a.w, a.n, a.k, a.ldw = weight.data_ptr(), weight.shape[0], weight.shape[1], weight.stride(0)
    if bias is not None:
        _dev("bias", bias, torch.bfloat16)
        a.bias = bias.data_ptr()
    norm = hidden is not None
    if norm:
        _dev("hidden", hidden, torch.float32)
        _dev("norm_weight", norm_weight, torch.bfloat16)
        if hidden.shape[1] != a.k or norm_weight.numel() != a.k:
            raise KernelError("skinny_gemm: hidden/norm_weight widths do not match the weight's K")
        a.hidden, a.norm_w, a.eps, a.m = hidden.data_ptr(), norm_weight.data_ptr(), eps, hidden.shape[0]
    else:
        _dev("x", x, torch.bfloat16, contiguous=False)
        if x.shape[1] != a.k or x.stride(1) != 1:
            raise KernelError("skinny_gemm: x width does not match the weight's K")
        a.x, a.ldx, a.m = x.data_ptr(), x.stride(0), x.shape[0]
    if epilogue == EPI_PLAIN:
        _dev("out", out, None, contiguous=False)
        if out.shape != (a.m, a.n) or out.dtype not in (torch.bfloat16, torch.float32):
            raise KernelError("skinny_gemm: out must be [m, N] bf16 or float32")
        a.out, a.ldo, a.out_f32 = out.data_ptr(), out.stride(0), int(out.dtype == torch.float32)
    elif epilogue == EPI_RESIDUAL:
        _dev("residual", residual, torch.float32)
        if residual.shape != (a.m, a.n):
            raise KernelError("skinny_gemm: residual must be [m, N] float32")
        a.residual = residual.data_ptr()
    elif epilogue == EPI_SWIGLU:
        _dev("out", out, torch.bfloat16)
        a.inter = a.n // 2
        if out.shape != (a.m, a.inter):
            raise KernelError("skinny_gemm: out must be [m, N / 2] bf16")
        a.out, a.ldo = out.data_ptr(), out.stride(0)
    elif epilogue == EPI_QKV:
        site = qkv["site"]
        _dev("q_out", qkv["q_out"], torch.bfloat16)
        _dev("cache", site.storage, torch.bfloat16)
        a.n_heads, a.kv_heads, a.head_dim = qkv["n_heads"], site.kv_heads, site.head_dim
        a.rot_dim, a.write_cache = qkv["rot_dim"], int(bool(qkv["write_cache"]))
        a.inv_freq = 0 if qkv["inv_freq"] is None else qkv["inv_freq"].data_ptr()
        a.tok_pos, a.tok_seq, a.slots = qkv["tok_pos"].data_ptr(), qkv["tok_seq"].data_ptr(), qkv["slots"].data_ptr()
        a.q_out, a.kv_base, a.table = qkv["q_out"].data_ptr(), site.storage.data_ptr(), site.table.data_ptr()
        a.page_elems, a.table_stride, a.err = site.page_elems, site.table_stride, qkv["err"].data_ptr()
        if qkv["q_out"].shape != (a.m, a.n_heads * a.head_dim):
            raise KernelError("skinny_gemm: q_out must be [m, n_heads * head_dim]")
    else:
        raise KernelError(f"skinny_gemm: unknown epilogue {epilogue}")
    if not a.err:
        a.err = (err if err is not None else _err_word_for(weight.device)).data_ptr()
    return a, norm


def skinny_gemm(epilogue: int, weight: torch.Tensor, **tensors) -> None:
    """One fused product for up to 16 token rows. Input rows are either `x` [m, K] bf16, or the float32 residual
    stream `hidden` [m, K] normalised on the fly with `norm_weight`, `eps`. Keywords: x | hidden, norm_weight, eps;
    bias; out (PLAIN, SWIGLU); residual (RESIDUAL); err; see csrc/skinny_gemm.cu for the epilogues.
    qkv (EPI_QKV): dict(n_heads, site=KvSiteArgs, inv_freq, rot_dim, tok_pos, tok_seq, slots, q_out, write_cache, err)."""
    a, norm = _skinny_args(epilogue, weight, **tensors)
    code = library("skinny_gemm").qf_skinny_gemm(_I(epilogue), _I(int(norm)), ctypes.byref(a), _stream())
    if code == 1:  # cudaErrorInvalidValue: a shape the kernel does not take
        raise KernelError(f"skinny_gemm: shape m={a.m} n={a.n} k={a.k} (epilogue {epilogue}) is not supported; "
                          "use the unfused kernels")
    _check(code, "skinny_gemm")


WIDE_MAX_ROWS = 64
_wide_answers: dict = {}


def wide_gemm_takes(epilogue: int, weight: torch.Tensor, **tensors) -> bool:
    """Whether `wide_gemm` runs this product (up to 64 token rows `x`; the library's own planning, launching nothing)."""
    x = tensors.get("x")
    if x is None or not (weight.is_cuda and weight.dtype == torch.bfloat16 and x.dtype == torch.bfloat16):
        return False
    qkv = tensors.get("qkv") or {}
    site = qkv.get("site")
    key = (weight.device.index, epilogue, tuple(weight.shape), weight.stride(0), tuple(x.shape), x.stride(0),
           weight.data_ptr() % 16, x.data_ptr() % 16, tensors.get("bias") is not None, qkv.get("n_heads"),
           None if site is None else (site.kv_heads, site.head_dim), qkv.get("rot_dim"), qkv.get("inv_freq") is not None)
    answer = _wide_answers.get(key)
    if answer is None:
        try:
            a, _ = _skinny_args(epilogue, weight, **tensors)
        except KernelError:
            return False
        with torch.cuda.device(weight.device):
            answer = library("wide_gemm").qf_wide_gemm_takes(_I(epilogue), ctypes.byref(a)) != 0
        _wide_answers[key] = answer
    return answer


def wide_gemm_takes_rows(epilogue: int, m: int, weight: torch.Tensor) -> bool:
    """`wide_gemm_takes` for planning, before the step's tensors exist: `m` contiguous, aligned token rows against
    `weight`, for the epilogues without further arguments (EPI_RESIDUAL, EPI_SWIGLU, EPI_PLAIN)."""
    if not (weight.is_cuda and weight.dtype == torch.bfloat16) or epilogue == EPI_QKV:
        return False
    key = (weight.device.index, epilogue, tuple(weight.shape), weight.stride(0), m, weight.data_ptr() % 16)
    answer = _wide_answers.get(key)
    if answer is None:
        a = _SkinnyArgs()
        a.w, a.n, a.k, a.ldw = weight.data_ptr(), weight.shape[0], weight.shape[1], weight.stride(0)
        a.x, a.ldx, a.m = 256, weight.shape[1], m          # only the alignment of the rows is looked at
        a.inter = a.n // 2 if epilogue == EPI_SWIGLU else 0
        with torch.cuda.device(weight.device):
            answer = library("wide_gemm").qf_wide_gemm_takes(_I(epilogue), ctypes.byref(a)) != 0
        _wide_answers[key] = answer
    return answer


def residual_product_way(m: int, weight: torch.Tensor) -> str:
    """How `m` token rows (64 at most) are multiplied by `weight` [N, K] and added into the residual stream fastest, by
    measurement on a B200 (`python -m qwenforge_b200.measure products`, Qwen2.5 0.5B / 3B / 7B sizes).
    Up to 16 rows the choice is between the two kernels that add in place: "skinny" (the mma.sync streamer) up to 8 rows
    while the weight is under 20 MB (0.5B: 3.0 and 4.8 microseconds against 3.4 and 5.5 on the tcgen05 streamer; 7B's
    26 MB output projection: 9.0 against 8.0), "wide" (the tcgen05 streamer) beyond (16 rows: 3.4 / 5.5 against 4.1 /
    6.6 at 0.5B, 14.9 against 16.2 at 3B's down product, 25.8 against 50 at 7B's).
    From 17 rows on the other way is the library product, whose result the next norm kernel adds at no cost: "wide" is
    the faster one only for products with a long K (a feed-forward's down product: 7.2 against 9 microseconds at 0.5B
    with 64 rows, 29.5 against 31.6 at 7B; an output projection: 4.6 against 3.1), so it needs K >= 2 N there.
    "unfused" (library product, addition by the next norm) is what remains."""
    size = weight.numel() * weight.element_size()
    skinny = m <= SKINNY_MAX_ROWS and skinny_gemm_takes(m, weight, EPI_RESIDUAL, False)
    wide = m <= WIDE_MAX_ROWS and wide_gemm_takes_rows(EPI_RESIDUAL, m, weight)
    if m > SKINNY_MAX_ROWS:
        return "wide" if wide and weight.shape[1] >= 2 * weight.shape[0] else "unfused"
    if skinny and (not wide or (m <= 8 and size < 20e6)):
        return "skinny"
    return "wide" if wide else "unfused"


def wide_gemm(epilogue: int, weight: torch.Tensor, **tensors) -> None:
    """One fused product for up to 64 token rows on the tcgen05 tensor cores (csrc/wide_gemm.cu): the keywords of
    `skinny_gemm`, with the input rows always given as `x` [m, K] bf16 (already normalised)."""
    a, norm = _skinny_args(epilogue, weight, **tensors)
    if norm:
        raise KernelError("wide_gemm: the input rows must be given as x (normalise them first)")
    code = library("wide_gemm").qf_wide_gemm(_I(epilogue), ctypes.byref(a), _stream())
    if code == 1:
        raise KernelError(f"wide_gemm: shape m={a.m} n={a.n} k={a.k} (epilogue {epilogue}) is not supported; "
                          "use the unfused kernels")
    if code == 801:
        raise KernelError("wide_gemm: the driver offers no tensor-map encoder (cuTensorMapEncodeTiled)")
    _check(code, "wide_gemm")


class FusedProduct:
    """One fused product, described but not run: the epilogue, the weight and the keywords of `skinny_gemm`. Parts hand
    these out so that whoever arranges them can run several as one chain (`skinny_chain`) or each alone (`run`)."""
    __slots__ = ("epilogue", "weight", "tensors")

    def __init__(self, epilogue: int, weight: torch.Tensor, **tensors):
        self.epilogue, self.weight, self.tensors = epilogue, weight, tensors

    def run(self) -> None:
        skinny_gemm(self.epilogue, self.weight, **self.tensors)


class _ChainProduct(ctypes.Structure):
    _fields_ = [("epilogue", _I), ("norm", _I), ("a", _SkinnyArgs)]


CHAIN_MAX_PRODUCTS = 4
_chain_answers: dict = {}


def _chain_array(products):
    array = (_ChainProduct * len(products))()
    for i, product in enumerate(products):
        a, norm = _skinny_args(product.epilogue, product.weight, **product.tensors)
        array[i].epilogue, array[i].norm, array[i].a = product.epilogue, int(norm), a
    return array


def skinny_chain_takes(products) -> bool:
    """Whether `skinny_chain` runs these products as ONE persistent kernel (the library's own planning, launching nothing)."""
    if not 1 <= len(products) <= CHAIN_MAX_PRODUCTS:
        return False
    key = tuple((p.epilogue, p.weight.shape, p.weight.stride(0), "hidden" in p.tensors,
                 (p.tensors.get("hidden") if "hidden" in p.tensors else p.tensors["x"]).shape[0],
                 p.tensors["x"].stride(0) if "x" in p.tensors else 0) for p in products) + (products[0].weight.device.index,)
    answer = _chain_answers.get(key)
    if answer is None:
        with torch.cuda.device(products[0].weight.device):
            answer = library("skinny_chain").qf_skinny_chain_takes(_I(len(products)), _chain_array(products)) != 0
        _chain_answers[key] = answer
    return answer


def skinny_chain(products, sync: torch.Tensor, err: torch.Tensor) -> None:
    """Runs up to four fused products, each reading what the one before wrote, as one persistent kernel whose blocks
    stream the weights of all of them without a pause (csrc/skinny_chain.cu). `sync`: two int32 words, zero when first
    used, that belong to this stream's chains."""
    _dev("sync", sync, torch.int32)
    _dev("err", err, torch.int32)
    if sync.numel() < 2:
        raise KernelError("skinny_chain: sync must hold two words")
    code = library("skinny_chain").qf_skinny_chain(_I(len(products)), _chain_array(products), _ptr(sync), _ptr(err), _stream())
    if code == 1:
        raise KernelError("skinny_chain: these products do not fit the chain kernel; run them one by one")
    _check(code, "skinny_chain")


def skinny_chain_repeated(products, repeats: int, steps, sync: torch.Tensor, err: torch.Tensor) -> None:
    """A measuring aid: the chain run `repeats` times over inside ONE launch. steps: per product the elements by which
    its weight, its bias and its norm weight advance per repeat (three lists; stacked tensors); all else is shared."""
    flat = (ctypes.c_longlong * 12)(*([0] * 12))
    for kind, values in enumerate(steps):
        for i, value in enumerate(values):
            flat[4 * kind + i] = int(value)
    code = library("skinny_chain").qf_skinny_chain_repeated(_I(len(products)), _chain_array(products), _I(repeats), flat,
                                                            _ptr(sync), _ptr(err), _stream())
    if code == 1:
        raise KernelError("skinny_chain: these products do not fit the chain kernel; run them one by one")
    _check(code, "skinny_chain_repeated")


def residual_add(hidden: torch.Tensor, delta: torch.Tensor) -> None:
    """hidden (float32) += delta, in place."""
    _dev("hidden", hidden, torch.float32)
    _dev("delta", delta)
    if delta.shape != hidden.shape:
        raise KernelError("residual_add: shapes differ")
    _check(library("norm").qf_residual_add(_I(_is_bf16(delta.dtype)), _ptr(hidden), _ptr(delta), _LL(hidden.numel()),
                                           _stream()), "residual_add")


# ---------------------------------------------------------------------------------------------- tcgen05 products

TC_PLAIN, TC_SWIGLU = 0, 1


def tc_gemm_takes(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether the tcgen05 kernel takes x [M, K] against weight [N, K]: bf16, K and the row strides multiples of 8."""
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.stride(1) == 1 and weight.stride(1) == 1
            and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


class _TcQkvArgs(ctypes.Structure):
    _fields_ = [("bias", ctypes.c_void_p), ("angles", ctypes.c_void_p), ("tok_pos", ctypes.c_void_p), ("tok_seq", ctypes.c_void_p),
                ("slots", ctypes.c_void_p), ("q_out", ctypes.c_void_p), ("kv_base", ctypes.c_void_p), ("table", ctypes.c_void_p),
                ("page_elems", ctypes.c_longlong), ("table_stride", _I), ("n_heads", _I), ("kv_heads", _I), ("head_dim", _I),
                ("write_cache", _I)]


def rope_table(tok_pos: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """The rotation angles of a step's tokens, [tokens, rot_dim / 2, 2] float32 (cos, sin): made once, read by every layer."""
    _dev("tok_pos", tok_pos, torch.int32)
    _dev("inv_freq", inv_freq, torch.float32)
    table = torch.empty((tok_pos.numel(), inv_freq.numel(), 2), dtype=torch.float32, device=tok_pos.device)
    _check(library("rope_cache").qf_rope_table(_ptr(tok_pos), _ptr(inv_freq), _I(tok_pos.numel()), _I(inv_freq.numel()), _ptr(table),
                                               _stream()), "rope_table")
    return table


TC_QKV_HEAD_DIMS = (32, 64, 128)


def tc_gemm_qkv_takes(x: torch.Tensor, weight: torch.Tensor, head_dim: int) -> bool:
    """Whether `tc_gemm_qkv` takes these operands: what `tc_gemm_takes` asks, and whole heads per tile of 128 columns."""
    return head_dim in TC_QKV_HEAD_DIMS and tc_gemm_takes(x, weight)


def tc_gemm_qkv(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], angles: Optional[torch.Tensor],
                tok_seq: torch.Tensor, tok_pos: torch.Tensor, slots: torch.Tensor, n_heads: int, q_out: torch.Tensor,
                site: KvSiteArgs, write_cache: bool, err: torch.Tensor) -> None:
    """The query/key/value product of many token rows on the tcgen05 tensor cores with its bias, the rotation of q and k
    heads by the tokens' angles (`rope_table`; None: no rotation) and the writes in its epilogue: q to `q_out`
    [tokens, n_heads * head_dim], k and v to each token's place in its sequence's cache page."""
    _dev("x", x, torch.bfloat16, contiguous=False)
    _dev("weight", weight, torch.bfloat16, contiguous=False)
    _dev("q_out", q_out, torch.bfloat16)
    _dev("cache", site.storage, torch.bfloat16)
    d = site.head_dim
    m, k = x.shape
    if weight.shape != ((n_heads + 2 * site.kv_heads) * d, k) or q_out.shape != (m, n_heads * d):
        raise KernelError("tc_gemm_qkv: weight must be [(n_heads + 2 kv_heads) * head_dim, K] and q_out [tokens, n_heads * head_dim]")
    if not tc_gemm_qkv_takes(x, weight, d):
        raise KernelError(f"tc_gemm_qkv: head_dim {d} or the operands' alignment is not taken (head sizes {TC_QKV_HEAD_DIMS})")
    if angles is not None and (angles.dtype != torch.float32 or angles.shape != (m, d // 2, 2) or not angles.is_contiguous()):
        raise KernelError("tc_gemm_qkv: angles must be float32 [tokens, head_dim / 2, 2] (the whole head is rotated)")
    a = _TcQkvArgs()
    a.bias = None if bias is None else bias.data_ptr()
    a.angles = None if angles is None else angles.data_ptr()
    a.tok_pos, a.tok_seq, a.slots = tok_pos.data_ptr(), tok_seq.data_ptr(), slots.data_ptr()
    a.q_out, a.kv_base, a.table = q_out.data_ptr(), site.storage.data_ptr(), site.table.data_ptr()
    a.page_elems, a.table_stride = site.page_elems, site.table_stride
    a.n_heads, a.kv_heads, a.head_dim, a.write_cache = n_heads, site.kv_heads, d, int(bool(write_cache))
    code = library("tc_gemm").qf_tc_gemm_qkv(_ptr(x), _I(x.stride(0)), _ptr(weight), _I(weight.stride(0)), _I(m), _I(k),
                                             ctypes.byref(a), _ptr(err), _stream())
    if code == 801:
        raise KernelError("tc_gemm_qkv: the driver offers no tensor-map encoder (cuTensorMapEncodeTiled)")
    _check(code, "tc_gemm_qkv")


def tc_gemm_is_persistent(epilogue: int, m: int, n: int) -> bool:
    """Whether `tc_gemm` runs x [m, K] against weight [n, K] in its persistent kernel (tiles for every SM)."""
    return library("tc_gemm").qf_tc_gemm_is_persistent(_I(epilogue), _I(m), _I(n)) != 0


def tc_gemm(epilogue: int, x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, err: Optional[torch.Tensor] = None) -> None:
    """out = x @ weight.T on the tcgen05 tensor cores (bf16 in, float32 accumulate in tensor memory, bf16 out).
    TC_SWIGLU: weight = [gate rows | up rows], out [M, N / 2] = silu(x gate^T) * (x up^T)."""
    _dev("x", x, torch.bfloat16, contiguous=False)
    _dev("weight", weight, torch.bfloat16, contiguous=False)
    _dev("out", out, torch.bfloat16, contiguous=False)
    m, k = x.shape
    n = weight.shape[0]
    cols = n // 2 if epilogue == TC_SWIGLU else n
    if weight.shape[1] != k or out.shape != (m, cols) or out.stride(1) != 1:
        raise KernelError(f"tc_gemm: shapes {tuple(x.shape)} x {tuple(weight.shape)}^T -> {tuple(out.shape)} do not agree")
    if not tc_gemm_takes(x, weight) or out.stride(0) % 8 or out.data_ptr() % 16:
        raise KernelError("tc_gemm: operands must be bf16 with K and row strides multiples of 8 and 16-byte aligned")
    err = err if err is not None else _err_word_for(x.device)
    code = library("tc_gemm").qf_tc_gemm(_I(epilogue), _ptr(x), _I(x.stride(0)), _ptr(weight), _I(weight.stride(0)), _ptr(out),
                                         _I(out.stride(0)), _I(m), _I(n), _I(k), _ptr(err), _stream())
    if code == 801:
        raise KernelError("tc_gemm: the driver offers no tensor-map encoder (cuTensorMapEncodeTiled)")
    _check(code, "tc_gemm")
