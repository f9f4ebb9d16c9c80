"""Grouped-query softmax attention over the cache (student_engine.py:556-599, :795-832).

  qkv = x Wqkv^T + bqkv            one product on the row-concatenated q, k, v weights (:505-520)
  q, k rotated by position         the position part; fused into the cache-write kernel when it is rotary
  k, v appended to the cache       at the token's own position of its own sequence
  ctx = softmax(q k^T * scale) v   query head i reads kv head i // (NH / KVH); key j visible iff
                                   max(0, p - window + 1) <= j <= p for a query at position p
  out = ctx Wo^T (+ bo)

Nothing here is specific to one model: head counts, head size, biases, scale, window and the
position part all come from the spec. A step's queries attend to the cache only, which already
holds the step's own keys: whole prompts, continuations and single tokens are the same code.
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache import PAGE_TOKENS, KvNeed
from .base import Mixer, TensorSpec
from .registry import build_part, register_part


# Fewest new tokens of a step, by head size, from which the tcgen05 prefill attention runs instead of the mma.sync one.
# Measured on one prompt (`python -m qwenforge_b200.measure attention`): head size 64, 14 heads: 17 against 21
# microseconds at 1,024 tokens, 27 against 42 at 2,048, 72 against 116 at 4,096, 199 against 415 at 8,192 (at 512 tokens
# 15 against 13); head size 128, 16 heads: 16 against 17 at 512 tokens, 24 against 36 at 1,024, 52 against 72 at 2,048,
# 140 against 245 at 4,096. Below, its tiles of 128 rows are too few to fill the SMs.
TC_PREFILL_MIN_TOKENS = {64: 1024, 128: 512}


class GqaAttention(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, qkv_bias, out_bias, scale, window, position (PartSpec | None).
    tensors: q_weight, k_weight, v_weight, o_weight (+ q_bias, k_bias, v_bias, o_bias when enabled)."""

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["num_heads"])
        self.n_kv = int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.qkv_bias = bool(p.get("qkv_bias", False))
        self.out_bias = bool(p.get("out_bias", False))
        self.scale = float(p.get("scale") or self.head_dim ** -0.5)
        self.window = int(p.get("window") or 0)
        if self.n_heads % self.n_kv:
            raise ValueError(f"gqa_attention: {self.n_heads} heads are not divisible by {self.n_kv} kv heads")
        if self.head_dim > 256:
            raise ValueError(f"gqa_attention: head_dim {self.head_dim} > 256 is not supported by the attention kernels")
        self.position = build_part("position", p["position"]) if p.get("position") is not None else None
        self.q_width = self.n_heads * self.head_dim
        self.kv_width = self.n_kv * self.head_dim
        self.qkv_weight = self.qkv_bias_t = self.o_weight = self.o_bias_t = None

    def sub_parts(self):
        return [self.position] if self.position is not None else []

    def tensor_specs(self):
        specs = [
            TensorSpec(self.file_name("q_weight"), (self.q_width, self.hidden)),
            TensorSpec(self.file_name("k_weight"), (self.kv_width, self.hidden)),
            TensorSpec(self.file_name("v_weight"), (self.kv_width, self.hidden)),
            TensorSpec(self.file_name("o_weight"), (self.hidden, self.q_width)),
        ]
        if self.qkv_bias:
            specs += [
                TensorSpec(self.file_name("q_bias"), (self.q_width,), init="bias"),
                TensorSpec(self.file_name("k_bias"), (self.kv_width,), init="bias"),
                TensorSpec(self.file_name("v_bias"), (self.kv_width,), init="bias"),
            ]
        if self.out_bias:
            specs.append(TensorSpec(self.file_name("o_bias"), (self.hidden,), init="bias"))
        return specs

    def kernel_libraries(self, dtype):
        libs = {"rope_cache", "attention_generic"}
        if dtype == torch.float32:
            libs.add("gemm_f32")
        elif self.head_dim in ops.FAST_ATTENTION_HEAD_DIMS:
            libs |= {"attention_decode", "attention_prefill", "skinny_gemm", "wide_gemm", "fold_project"}
            if self.head_dim in ops.TC_ATTENTION_HEAD_DIMS:
                libs.add("attention_prefill_tc")
        return libs

    def cache_need(self):
        return KvNeed(self.n_kv, self.head_dim, self.window)

    def bind(self, tensors, dtype, device):
        t = lambda logical: tensors[self.file_name(logical)]
        self.qkv_weight = torch.cat((t("q_weight"), t("k_weight"), t("v_weight")), dim=0).contiguous()
        if self.qkv_bias:
            self.qkv_bias_t = torch.cat((t("q_bias"), t("k_bias"), t("v_bias")), dim=0).contiguous()
        self.o_weight = t("o_weight")
        if self.out_bias:
            self.o_bias_t = t("o_bias")

    def step_weights(self):
        return [t for t in (self.qkv_weight, self.qkv_bias_t, self.o_weight, self.o_bias_t) if t is not None]

    def forward(self, x, ctx, site, writes_cache):
        n = x.shape[0]
        fast = (ctx.attention == "auto" and x.dtype == torch.bfloat16
                and self.head_dim in ops.FAST_ATTENTION_HEAD_DIMS)
        plan = self.decode_plan(ctx) if fast and ctx.is_decode else None
        rotary = self.position.fused_rotary() if self.position is not None else None
        # (The product with bias, rotation and cache write in its epilogue, `ops.tc_gemm_qkv`, was measured inside the
        # prompt graph of 2,048 tokens at Qwen2.5-0.5B sizes: 2.88 ms for the step against 2.76 with the library product
        # and the rotation kernel; it is not used here.)
        late_bias = self.position is None or rotary is not None  # the kernel that rotates and stores adds the bias
        qkv = ops.linear(x, self.qkv_weight, None if late_bias else self.qkv_bias_t)
        if self.position is not None and rotary is None:
            q_view = qkv[:, :self.q_width].view(n, self.n_heads, self.head_dim)
            k_view = qkv[:, self.q_width:self.q_width + self.kv_width].view(n, self.n_kv, self.head_dim)
            self.position.apply(q_view, k_view, ctx)
        inv_freq, rot_dim = rotary if rotary is not None else (None, 0)
        q = torch.empty((n, self.q_width), dtype=x.dtype, device=x.device)
        args = ops.KvSiteArgs(site.storage, site.table, self.n_kv, self.head_dim)
        ops.rope_cache_write(qkv, ctx.tok_seq, ctx.tok_pos, ctx.slots, inv_freq, rot_dim, self.n_heads, q, args,
                             writes_cache, ctx.err, bias=self.qkv_bias_t if late_bias else None)
        attended = torch.empty_like(q)
        if fast and ctx.is_decode:
            ops.attention_decode(q, attended, ctx.cu_q, ctx.tok_pos, ctx.slots, args, self.n_heads, ctx.n_seqs,
                                 self.scale, self.window, self.decode_splits(ctx), ctx.decode_scratch, ctx.err, plan)
        elif fast:
            # the tcgen05 kernel works on blocks of 128 query rows, a long chain of pages per block: it pays for steps
            # with many rows
            least = TC_PREFILL_MIN_TOKENS.get(self.head_dim)
            prefill = (ops.attention_prefill_tc if least is not None and n >= least and ctx.max_q_len >= 128
                       else ops.attention_prefill)
            prefill(q, attended, ctx.cu_q, ctx.tok_pos, ctx.slots, args, self.n_heads, ctx.n_seqs,
                    ctx.max_q_len, self.scale, self.window, ctx.err, max_kv_len=ctx.max_kv_len)
        else:
            ops.attention_generic(q, attended, ctx.cu_q, ctx.tok_pos, ctx.slots, args, self.n_heads, ctx.n_seqs,
                                  ctx.max_q_len, self.scale, self.window, ctx.err, scratch=ctx.decode_scratch,
                                  max_kv_len=ctx.max_kv_len)
        return ops.linear(attended, self.o_weight, self.o_bias_t)

    # ---- the form for decode steps of up to 64 sequences that works on the residual stream in place: the norm, bias,
    # rotation and cache write ride on the QKV product and the addition on the output projection wherever a kernel of
    # this library takes the sizes and is the faster way by measurement; each product chooses for itself.
    def _ways(self, ctx):
        rows = ctx.n_tokens
        rotary = self.position.fused_rotary() if self.position is not None else None
        qkv = "unfused"
        if rows <= ops.SKINNY_MAX_ROWS and ops.skinny_gemm_takes(rows, self.qkv_weight, ops.EPI_QKV, True, n_heads=self.n_heads,
                                                                 kv_heads=self.n_kv, head_dim=self.head_dim,
                                                                 rot_dim=rotary[1] if rotary else 0):
            qkv = "skinny"
        return qkv, ops.residual_product_way(rows, self.o_weight)

    def fused_takes(self, ctx) -> bool:
        if not (ctx.attention == "auto" and ctx.is_decode and ctx.dtype == torch.bfloat16 and ctx.n_tokens <= ops.WIDE_MAX_ROWS
                and self.head_dim in ops.FAST_ATTENTION_HEAD_DIMS and not self.out_bias):
            return False
        rotary = self.position.fused_rotary() if self.position is not None else None
        if self.position is not None and (rotary is None or rotary[1] != self.head_dim):
            return False
        return self._ways(ctx) != ("unfused", "unfused")

    def fused_forward(self, hidden, rms, ctx, site, writes_cache, delta=None):
        n = hidden.shape[0]
        qkv_way, o_way = self._ways(ctx)
        plan = self.decode_plan(ctx)
        inv_freq, rot_dim = self.position.fused_rotary() if self.position is not None else (None, 0)
        args = ops.KvSiteArgs(site.storage, site.table, self.n_kv, self.head_dim)
        q = torch.empty((n, self.q_width), dtype=torch.bfloat16, device=hidden.device)
        if qkv_way == "skinny":
            if delta is not None:
                ops.residual_add(hidden, delta)
            ops.skinny_gemm(ops.EPI_QKV, self.qkv_weight, hidden=hidden, norm_weight=rms[0], eps=rms[1],
                            bias=self.qkv_bias_t,
                            qkv=dict(n_heads=self.n_heads, site=args, inv_freq=inv_freq, rot_dim=rot_dim, tok_pos=ctx.tok_pos,
                                     tok_seq=ctx.tok_seq, slots=ctx.slots, q_out=q, write_cache=writes_cache, err=ctx.err))
        else:
            x = torch.empty(hidden.shape, dtype=torch.bfloat16, device=hidden.device)
            ops.add_rms_norm(hidden, delta, rms[0], rms[1], x)   # the norm kernel adds the pending delta on its way
            ops.rope_cache_write(ops.linear(x, self.qkv_weight), ctx.tok_seq, ctx.tok_pos, ctx.slots, inv_freq, rot_dim,
                                 self.n_heads, q, args, writes_cache, ctx.err, bias=self.qkv_bias_t)
        n_splits = self.decode_splits(ctx)
        if (o_way == "skinny" and n == ctx.n_seqs and ops.fold_project_pays(n, self.o_weight)
                and ops.fold_project_takes(n, self.o_weight, hidden, self.n_heads, self.head_dim)):
            # the attention kernel stops at its runs' partial results; the projection folds them on its way in
            ops.attention_decode(q, None, ctx.cu_q, ctx.tok_pos, ctx.slots, args, self.n_heads, ctx.n_seqs, self.scale,
                                 self.window, n_splits, ctx.decode_scratch, ctx.err, plan, fold_later=True)
            ops.fold_project(plan, ctx.decode_scratch, self.o_weight, hidden, self.n_heads, self.head_dim, n_splits)
            return
        attended = torch.empty_like(q)
        ops.attention_decode(q, attended, ctx.cu_q, ctx.tok_pos, ctx.slots, args, self.n_heads, ctx.n_seqs,
                             self.scale, self.window, n_splits, ctx.decode_scratch, ctx.err, plan)
        if o_way == "skinny":
            ops.skinny_gemm(ops.EPI_RESIDUAL, self.o_weight, x=attended, residual=hidden)
        elif o_way == "wide":
            ops.wide_gemm(ops.EPI_RESIDUAL, self.o_weight, x=attended, residual=hidden, err=ctx.err)
        else:
            ops.residual_add(hidden, ops.linear(attended, self.o_weight))

    def decode_plan(self, ctx) -> torch.Tensor:
        """Which block of the decode attention takes which run of which sequence: made once per step, by the first
        layer of this shape that runs, and shared through the step's memo by the others."""
        n_splits = self.decode_splits(ctx)
        key = ("gqa_attention.decode_plan", self.n_kv, self.n_heads, self.head_dim, self.window, n_splits)
        memo = ctx.step_memo if ctx.step_memo is not None else {}
        plan = memo.get(key)
        if plan is None:
            plan = memo[key] = ops.attention_decode_plan(ctx.cu_q, ctx.tok_pos, ctx.slots, self.n_kv, self.head_dim,
                                                         self.n_heads, ctx.n_seqs, self.window, n_splits, ctx.decode_scratch)
        return plan

    def decode_splits(self, ctx) -> int:
        """The most blocks that may share one (sequence, kv head): a block's warps take one page each
        (`ops.attention_decode_warps`), so at most one split per that many pages of the longest sequence that the step allows.
        How many of them a sequence gets is the kernel's decision, from the lengths on the device; this number sizes
        its grid and scratch and depends on the batch's shape only (fixed inside a captured graph)."""
        span = ctx.max_kv_len if self.window <= 0 else min(ctx.max_kv_len, self.window + PAGE_TOKENS)
        pages = max(1, -(-span // PAGE_TOKENS))
        warps = ops.attention_decode_warps(self.head_dim)
        return max(1, min(-(-pages // warps), 64))


register_part("mixer", "gqa_attention", GqaAttention)
