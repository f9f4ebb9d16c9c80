"""Kernel-level measurements: how the fused kernels of this library compare with one another and with the unfused
path (norm kernel + library product + elementwise kernel) on the products of one decoder layer, and how the prefill
attention kernels compare. Every figure is the mean of CUDA-graph replays timed with CUDA events, the kernels of
`repeat` layers (each with weights of its own, so nothing is served from L2 twice) back to back in one graph.

    python -m qwenforge_b200.measure products --preset qwen2.5-0.5b --rows 1,8,16,64
    python -m qwenforge_b200.measure chain    --preset qwen2.5-0.5b --rows 8
    python -m qwenforge_b200.measure phases   --preset qwen2.5-0.5b --rows 1,64
    python -m qwenforge_b200.measure attention --tokens 1024,2048,4096 --heads 14 --kv-heads 2 --head-dim 64
    python -m qwenforge_b200.measure decode-attention --lengths 4000,4000,4000,4000,4000,4000,4000,4000 --splits 8
    python -m qwenforge_b200.measure gemm --preset qwen2.5-0.5b --rows 2048,16384

products   per product of a layer (output projection, gate/up, down, query/key/value): the weight-streaming kernel of
           skinny_gemm.cu (rows <= 16), the tcgen05 kernel of wide_gemm.cu (rows <= 64; after the norm kernel where the
           product normalises its rows), and the unfused kernels
chain      the four products after attention as separate kernels, as ONE persistent kernel per layer
           (skinny_chain.cu), and all layers' products inside one launch (the persistent kernel's steady state)
phases     wide_gemm.cu's own time stamps: when a block's copies, products, exchange and epilogue end
attention  the mma.sync and the tcgen05 prefill attention on one prompt, with a tile's pages shared or not
decode-attention  the split-K decode attention's own time stamps (launched alone, cold caches): which runs the plan
           gives every sequence, and when a block's copies, pages, merge, ticket and fold end; with and without the
           projection that folds the partial results
gemm       a feed-forward's gate/up product on many rows: the library product, the library product and the gate kernel,
           this library's tcgen05 product (one tile per block, and persistent) plain and with the gate in its epilogue
"""
from __future__ import annotations

import argparse
import ctypes
import sys

import torch

from . import ops
from .cache import PAGE_TOKENS
from .config import preset_config
from .engine.graphs import capturing

NAMES = ("output projection (residual)", "gate/up (norm, SwiGLU)", "down (residual)", "query/key/value (norm, rotation, cache)")


class Pages:
    """A paged key/value store of `n_slots` sequences of up to `max_len` positions, pages in scrambled order."""

    def __init__(self, n_slots: int, max_len: int, kv_heads: int, head_dim: int, device, seed: int = 0):
        per_seq = (max_len + PAGE_TOKENS - 1) // PAGE_TOKENS
        g = torch.Generator().manual_seed(seed)
        self.storage = torch.zeros(n_slots * per_seq + 3, 2, kv_heads, PAGE_TOKENS, head_dim, dtype=torch.bfloat16, device=device)
        self.table = torch.randperm(n_slots * per_seq + 3, generator=g)[:n_slots * per_seq].to(torch.int32).view(n_slots, per_seq).to(device)
        self.kv_heads, self.head_dim = kv_heads, head_dim

    def args(self) -> ops.KvSiteArgs:
        return ops.KvSiteArgs(self.storage, self.table, self.kv_heads, self.head_dim)


def layer_products(rows: int, hidden: int, inter: int, heads: int, kv_heads: int, head_dim: int, seed: int = 0, device="cuda"):
    """The four products that follow a decode step's attention, as `ops.FusedProduct`s over random tensors: output
    projection into the stream, norm + gate/up + SwiGLU, down into the stream, norm + the next layer's QKV with
    rotation and cache write. Returns (products, state), state holding every tensor that a run changes."""
    g = torch.Generator().manual_seed(seed)
    rnd = lambda *shape, scale=1.0: (torch.randn(*shape, generator=g) * scale)
    stream = rnd(rows, hidden).to(device)
    attended = rnd(rows, heads * head_dim).to(torch.bfloat16).to(device)
    o_w = rnd(hidden, heads * head_dim, scale=0.05).to(torch.bfloat16).to(device)
    gu_w = rnd(2 * inter, hidden, scale=0.05).to(torch.bfloat16).to(device)
    down_w = rnd(hidden, inter, scale=0.05).to(torch.bfloat16).to(device)
    qkv_w = rnd((heads + 2 * kv_heads) * head_dim, hidden, scale=0.05).to(torch.bfloat16).to(device)
    qkv_b = rnd((heads + 2 * kv_heads) * head_dim).to(torch.bfloat16).to(device)
    n1 = (1 + 0.1 * rnd(hidden)).to(torch.bfloat16).to(device)
    n2 = (1 + 0.1 * rnd(hidden)).to(torch.bfloat16).to(device)
    pages = Pages(rows, 400, kv_heads, head_dim, device)
    act = torch.zeros(rows, inter, dtype=torch.bfloat16, device=device)
    q_out = torch.zeros(rows, heads * head_dim, dtype=torch.bfloat16, device=device)
    tok_seq = torch.arange(rows, dtype=torch.int32, device=device)
    tok_pos = torch.tensor([(37 * i + 63) % 390 for i in range(rows)], dtype=torch.int32, device=device)
    slots = torch.tensor([(rows - 1 - i) if i != 1 else -1 for i in range(rows)], dtype=torch.int32, device=device)
    inv_freq = (1.0 / (1e6 ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))).to(device)
    err = torch.zeros(1, dtype=torch.int32, device=device)
    products = [
        ops.FusedProduct(ops.EPI_RESIDUAL, o_w, x=attended, residual=stream),
        ops.FusedProduct(ops.EPI_SWIGLU, gu_w, hidden=stream, norm_weight=n1, eps=1e-6, out=act),
        ops.FusedProduct(ops.EPI_RESIDUAL, down_w, x=act, residual=stream),
        ops.FusedProduct(ops.EPI_QKV, qkv_w, hidden=stream, norm_weight=n2, eps=1e-6, bias=qkv_b,
                         qkv=dict(n_heads=heads, site=pages.args(), inv_freq=inv_freq, rot_dim=head_dim, tok_pos=tok_pos,
                                  tok_seq=tok_seq, slots=slots, q_out=q_out, write_cache=True, err=err)),
    ]
    return products, dict(stream=stream, act=act, q_out=q_out, cache=pages.storage, err=err)


def graph_time_us(fn, per: int, replays: int = 30) -> float:
    """Microseconds per unit of work: `fn` captured into a CUDA graph once, replayed `replays` times between events."""
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        fn()
        fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with capturing(graph, stream):
        fn()
    for _ in range(5):
        graph.replay()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(replays):
        graph.replay()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / replays / per * 1e3


def unfused(product: ops.FusedProduct, err: torch.Tensor) -> None:
    """The same product by the unfused kernels: norm kernel, library product, elementwise kernel."""
    t = product.tensors
    if "hidden" in t:
        x = torch.empty(t["hidden"].shape, dtype=torch.bfloat16, device=t["hidden"].device)
        ops.add_rms_norm(t["hidden"], None, t["norm_weight"], t["eps"], x)
    else:
        x = t["x"]
    y = ops.linear(x, product.weight)
    if product.epilogue == ops.EPI_SWIGLU:
        ops.swiglu(y, t["out"])
    elif product.epilogue == ops.EPI_QKV:
        q = t["qkv"]
        ops.rope_cache_write(y, q["tok_seq"], q["tok_pos"], q["slots"], q["inv_freq"], q["rot_dim"], q["n_heads"], q["q_out"],
                             q["site"], True, err, bias=t["bias"])
    else:
        ops.residual_add(t["residual"], y)


def wide_tensors(product: ops.FusedProduct, x: torch.Tensor) -> dict:
    """`product`'s keywords for wide_gemm, which wants its rows already normalised: `x` receives them."""
    t = dict(product.tensors)
    if "hidden" in t:
        for key in ("hidden", "norm_weight", "eps"):
            t.pop(key)
        t["x"] = x
    return t


def wide(product: ops.FusedProduct, x: torch.Tensor) -> None:
    """The product by wide_gemm.cu, after the norm kernel where the product normalises its rows."""
    t = product.tensors
    if "hidden" in t:
        ops.add_rms_norm(t["hidden"], None, t["norm_weight"], t["eps"], x)
    ops.wide_gemm(product.epilogue, product.weight, **wide_tensors(product, x))


def sizes_of(preset: str):
    c = preset_config(preset)
    return c.hidden_size, c.intermediate_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim


def measure_products(args) -> None:
    hidden, inter, heads, kv_heads, head_dim = sizes_of(args.preset)
    repeat = args.repeat
    for rows in args.rows:
        layers = [layer_products(rows, hidden, inter, heads, kv_heads, head_dim, seed=100 + i) for i in range(repeat)]
        err = layers[0][1]["err"]
        xs = [torch.randn(rows, hidden, device="cuda").bfloat16() for _ in range(repeat)]
        for i, name in enumerate(NAMES):
            line = f"{args.preset} rows {rows:3d} {name:42s}"
            if rows <= ops.SKINNY_MAX_ROWS:
                line += f" skinny {graph_time_us(lambda: [layers[l][0][i].run() for l in range(repeat)], repeat):7.2f} us"
            p0 = layers[0][0][i]
            if rows <= ops.WIDE_MAX_ROWS and ops.wide_gemm_takes(p0.epilogue, p0.weight, **wide_tensors(p0, xs[0])):
                line += f"  wide {graph_time_us(lambda: [wide(layers[l][0][i], xs[l]) for l in range(repeat)], repeat):7.2f} us"
            line += f"  unfused {graph_time_us(lambda: [unfused(layers[l][0][i], err) for l in range(repeat)], repeat):7.2f} us"
            if p0.epilogue == ops.EPI_SWIGLU and rows > ops.SKINNY_MAX_ROWS:
                # the norm kernel, then the many-row tcgen05 product with the gate in its epilogue (one tile per block here)
                def own(l):
                    t = layers[l][0][i].tensors
                    ops.add_rms_norm(t["hidden"], None, t["norm_weight"], t["eps"], xs[l])
                    ops.tc_gemm(ops.TC_SWIGLU, xs[l], layers[l][0][i].weight, t["out"], err)
                line += f"  tc_gemm {graph_time_us(lambda: [own(l) for l in range(repeat)], repeat):7.2f} us"
            print(line, flush=True)
        if int(err):
            raise RuntimeError(f"a kernel reported error word {int(err)}")


def measure_chain(args) -> None:
    hidden, inter, heads, kv_heads, head_dim = sizes_of(args.preset)
    repeat = args.repeat
    for rows in args.rows:
        layers = [layer_products(rows, hidden, inter, heads, kv_heads, head_dim, seed=100 + i) for i in range(repeat)]
        err = layers[0][1]["err"]
        sync = torch.zeros(2, dtype=torch.int32, device="cuda")
        if not ops.skinny_chain_takes(layers[0][0]):
            print(f"{args.preset} rows {rows}: the chain kernel does not take these products")
            continue
        for n in (1, 2, 3, 4):
            separate = graph_time_us(lambda: [p.run() for l in range(repeat) for p in layers[l][0][:n]], repeat)
            chained = graph_time_us(lambda: [ops.skinny_chain(layers[l][0][:n], sync, err) for l in range(repeat)], repeat)
            print(f"{args.preset} rows {rows}: first {n} products of a layer: separate kernels {separate:6.2f} us, one persistent kernel "
                  f"{chained:6.2f} us", flush=True)
        # the steady state: every layer's products inside ONE launch (stacked weights)
        products, _ = layer_products(rows, hidden, inter, heads, kv_heads, head_dim, seed=7)
        keep = []
        for p in products:
            stacked = p.weight.unsqueeze(0).repeat(repeat, 1, 1).contiguous()
            keep.append(stacked)
            p.weight = stacked[0]
            for key in ("bias", "norm_weight"):
                if key in p.tensors:
                    more = p.tensors[key].unsqueeze(0).repeat(repeat, 1).contiguous()
                    keep.append(more)
                    p.tensors[key] = more[0]
        for first, count in ((0, 4), (0, 1), (1, 1), (2, 1), (3, 1)):
            chosen = products[first:first + count]
            steps = [[p.weight.numel() for p in chosen], [p.tensors["bias"].numel() if "bias" in p.tensors else 0 for p in chosen],
                     [p.tensors["norm_weight"].numel() if "norm_weight" in p.tensors else 0 for p in chosen]]
            us = graph_time_us(lambda: ops.skinny_chain_repeated(chosen, repeat, steps, sync, err), repeat)
            what = "all four products" if count == 4 else NAMES[first]
            print(f"{args.preset} rows {rows}: {repeat} layers inside one launch, {what}: {us:6.2f} us per layer", flush=True)
        if int(err):
            raise RuntimeError(f"a kernel reported error word {int(err)}")


def measure_phases(args) -> None:
    from .csrc import library
    from .ops import kernels
    hidden, inter, heads, kv_heads, head_dim = sizes_of(args.preset)
    print("mean microseconds since the first block's entry: set-up done, the kernel before done, first stage arrived, "
          "products done, sums sent, sums arrived, epilogue done (and the last block's end)")
    for rows in args.rows:
        products, state = layer_products(rows, hidden, inter, heads, kv_heads, head_dim)
        x = torch.randn(rows, hidden, device="cuda").bfloat16()
        for i, name in enumerate(NAMES):
            p = products[i]
            a, _ = kernels._skinny_args(p.epilogue, p.weight, **wide_tensors(p, x))
            stamps = torch.zeros(1024, 8, dtype=torch.int64, device="cuda")
            for _ in range(3):
                stamps.zero_()
                torch.cuda.synchronize()
                code = library("wide_gemm").qf_wide_gemm_stamped(ctypes.c_int(p.epilogue), ctypes.byref(a),
                                                                 ctypes.c_void_p(stamps.data_ptr()), kernels._stream())
                torch.cuda.synchronize()
            if code:
                print(f"{args.preset} rows {rows} {name}: not taken (code {code})")
                continue
            st = stamps.cpu()
            st = st[st[:, 0] > 0]
            rel = (st - int(st[:, 0].min())).double() / 1e3
            print(f"{args.preset} rows {rows:3d} {name:42s} blocks {st.shape[0]:3d}: "
                  + " ".join(f"{float(rel[:, k].mean()):6.2f}" for k in range(1, 8)) + f"  ({float(rel[:, 7].max()):6.2f})", flush=True)


def measure_attention(args) -> None:
    heads, kv_heads, d = args.heads, args.kv_heads, args.head_dim
    for n in args.tokens:
        pages = Pages(1, n, kv_heads, d, "cuda", 1)
        pages.storage.copy_(torch.randn(pages.storage.shape, device="cuda").to(torch.bfloat16))
        q = torch.randn(n, heads * d, device="cuda").bfloat16()
        out = torch.empty_like(q)
        cu = torch.tensor([0, n], dtype=torch.int32, device="cuda")
        pos = torch.arange(n, dtype=torch.int32, device="cuda")
        slots = torch.zeros(1, dtype=torch.int32, device="cuda")
        err = torch.zeros(1, dtype=torch.int32, device="cuda")
        flops = 4 * heads * d * n * (n + 1) / 2
        variants = [("mma.sync, a tile's pages by one group of warps", ops.attention_prefill, 64),
                    ("mma.sync, as the model runs it", ops.attention_prefill, n)]
        if d in ops.TC_ATTENTION_HEAD_DIMS:
            variants += [("tcgen05, one block per tile", ops.attention_prefill_tc, 64),
                         ("tcgen05, as the model runs it", ops.attention_prefill_tc, n)]
        for name, fn, bound in variants:
            run = lambda: fn(q, out, cu, pos, slots, pages.args(), heads, 1, n, d ** -0.5, 0, err, max_kv_len=bound)
            for _ in range(3):
                run()
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(20):
                run()
            end.record()
            torch.cuda.synchronize()
            us = start.elapsed_time(end) / 20 * 1e3
            print(f"one prompt of {n} tokens, {heads}/{kv_heads} heads of {d}: {name:46s} {us:7.1f} us  {flops / us / 1e6:5.0f} TFLOP/s", flush=True)
        if int(err):
            raise RuntimeError(f"a kernel reported error word {int(err)}")


DECODE_PHASES = ["entry", "early copies issued", "the kernel before done", "first half page arrived", "pages done",
                 "warps merged", "ticket drawn / partial results written", "fold done"]


def measure_decode_attention(args) -> None:
    """Time stamps of the phases of the split-K decode attention's blocks (and of the projection that folds its partial
    results), launched alone on cold caches: --lengths gives the sequences' lengths, --heads/--kv-heads/--head-dim the
    shape, --splits the most runs per sequence."""
    from .csrc import library
    from .ops import kernels
    lib = library("attention_decode")
    lib.qf_attention_decode_plan_size.restype = ctypes.c_longlong
    heads, kv_heads, d, lengths, n_splits = args.heads, args.kv_heads, args.head_dim, args.lengths, args.splits
    n = len(lengths)
    pages = Pages(n, max(lengths), kv_heads, d, "cuda", 1)
    pages.storage.copy_(torch.randn(pages.storage.shape, device="cuda").to(torch.bfloat16))
    q = torch.randn(n, heads * d, device="cuda").bfloat16()
    out = torch.empty_like(q)
    cu = torch.arange(n + 1, dtype=torch.int32, device="cuda")
    pos = torch.tensor([length - 1 for length in lengths], dtype=torch.int32, device="cuda")
    slots = torch.arange(n, dtype=torch.int32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    scratch = ops.DecodeScratch("cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    site = pages.args()
    kvc = kv_heads * (-(-(heads // kv_heads) // 16))
    records = int(lib.qf_attention_decode_plan_size(n, kv_heads, heads, d, n_splits)) - (n + 3) // 4
    hidden = torch.zeros(n, heads * d, device="cuda")
    o_w = (torch.randn(heads * d, heads * d, device="cuda") * 0.05).bfloat16()
    folds = n <= 16 and ops.fold_project_takes(n, o_w, hidden, heads, d)
    for fold_later in ([False, True] if folds else [False]):
        stamps = torch.zeros(records * kvc, 8, dtype=torch.int64, device="cuda")
        for it in range(4):
            flush.fill_(it)
            stamps.zero_()
            plan = ops.attention_decode_plan(cu, pos, slots, kv_heads, d, heads, n, 0, n_splits, scratch)
            scratch.ensure(n, heads, n_splits, d, n * kvc)
            torch.cuda.synchronize()
            start, mid, end = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            start.record()
            kernels._check(lib.qf_attention_decode_stamped(
                kernels._ptr(q), kernels._ptr(out), kernels._ptr(cu), kernels._ptr(plan), kernels._ptr(site.storage),
                kernels._ptr(site.table), ctypes.c_longlong(site.page_elems), ctypes.c_int(site.table_stride),
                ctypes.c_int(kv_heads), ctypes.c_int(d), ctypes.c_int(heads), ctypes.c_int(n), ctypes.c_float(d ** -0.5),
                ctypes.c_int(0), ctypes.c_int(n_splits), ctypes.c_int(int(fold_later)), kernels._ptr(scratch.part_o),
                kernels._ptr(scratch.part_ml), kernels._ptr(scratch.counters), kernels._ptr(err),
                kernels._ptr(stamps), kernels._stream()), "attention_decode")
            mid.record()
            if fold_later:
                ops.fold_project(plan, scratch, o_w, hidden, heads, d, n_splits)
            end.record()
            torch.cuda.synchronize()
        if int(err):
            raise RuntimeError(f"a kernel reported error word {int(err)}")
        st = stamps.cpu()
        st = st[st[:, 0] > 0]
        t0 = int(st[:, 0].min())
        runs = plan.cpu().flatten()[:n].tolist()
        mb = sum(lengths) * kv_heads * d * 2 * 2 / 1e6
        how = "stopping at the partial results" if fold_later else "folding its partial results itself"
        print(f"{n} sequences of {min(lengths)} to {max(lengths)} tokens, {heads}/{kv_heads} heads of {d}, {how}: {st.shape[0]} blocks, "
              f"runs per sequence {runs}, {mb:.1f} MB of keys and values; launched alone on cold caches: "
              f"{start.elapsed_time(mid) * 1e3:.1f} us" + (f", then the projection that folds {mid.elapsed_time(end) * 1e3:.1f} us" if fold_later else ""))
        for k, name in enumerate(DECODE_PHASES):
            col = st[:, k]
            col = (col[col > 0] - t0).double() / 1e3
            if len(col):
                print(f"    {name:40s} mean {float(col.mean()):6.2f}  last {float(col.max()):6.2f} us  ({len(col)} blocks)")


def measure_gemm(args) -> None:
    from .csrc import library
    hidden, inter, _, _, _ = sizes_of(args.preset)
    switch = library("tc_gemm").qf_tc_gemm_set_persistent

    def timed(fn, n=30):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(n):
            fn()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / n * 1e3

    for rows in args.rows:
        x = (torch.randn(rows, hidden, device="cuda") * 0.5).bfloat16()
        w = (torch.randn(2 * inter, hidden, device="cuda") * 0.05).bfloat16()
        full = torch.empty(rows, 2 * inter, dtype=torch.bfloat16, device="cuda")
        act = torch.empty(rows, inter, dtype=torch.bfloat16, device="cuda")
        flops = 2 * rows * 2 * inter * hidden
        print(f"{args.preset} gate/up product, {rows} x {2 * inter} x {hidden}:")
        rate = lambda us: f"{us:8.1f} us {flops / us / 1e6:6.0f} TFLOP/s"
        print("  library product                                   " + rate(timed(lambda: torch.mm(x, w.t(), out=full))))
        print("  library product, then the gate kernel             " + rate(timed(lambda: (torch.mm(x, w.t(), out=full), ops.swiglu(full, act)))))
        try:
            for mode, name in ((0, "one tile per block"), (1, "persistent")):
                switch(ctypes.c_int(mode))
                print(f"  tcgen05 product, {name:19s}              " + rate(timed(lambda: ops.tc_gemm(ops.TC_PLAIN, x, w, full))))
                print(f"  tcgen05 product with the gate, {name:19s}" + rate(timed(lambda: ops.tc_gemm(ops.TC_SWIGLU, x, w, act))), flush=True)
        finally:
            switch(ctypes.c_int(1))
        print(f"  (the persistent kernel {'runs' if ops.tc_gemm_is_persistent(ops.TC_SWIGLU, rows, 2 * inter) else 'does not run: too few tiles'} at this size)")
        # the query/key/value product: library product and the rotation / cache-write kernel, against the tcgen05 product
        # with bias, rotation and cache write in its epilogue
        _, _, heads, kv_heads, head_dim = sizes_of(args.preset)
        n_qkv = (heads + 2 * kv_heads) * head_dim
        wq = (torch.randn(n_qkv, hidden, device="cuda") * 0.05).bfloat16()
        bq = torch.randn(n_qkv, device="cuda").bfloat16()
        pages = Pages(1, rows, kv_heads, head_dim, "cuda")
        tok_seq = torch.zeros(rows, dtype=torch.int32, device="cuda")
        tok_pos = torch.arange(rows, dtype=torch.int32, device="cuda")
        slots = torch.zeros(1, dtype=torch.int32, device="cuda")
        inv_freq = (1.0 / (1e6 ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))).cuda()
        q_out = torch.empty(rows, heads * head_dim, dtype=torch.bfloat16, device="cuda")
        qkv = torch.empty(rows, n_qkv, dtype=torch.bfloat16, device="cuda")
        err = torch.zeros(1, dtype=torch.int32, device="cuda")
        flops_q = 2 * rows * n_qkv * hidden
        rate_q = lambda us: f"{us:8.1f} us {flops_q / us / 1e6:6.0f} TFLOP/s"
        print(f"{args.preset} query/key/value product, {rows} x {n_qkv} x {hidden}:")
        print("  library product                                   " + rate_q(timed(lambda: torch.mm(x, wq.t(), out=qkv))))
        print("  library product, then rotation and cache write    " + rate_q(timed(lambda: (
            torch.mm(x, wq.t(), out=qkv), ops.rope_cache_write(qkv, tok_seq, tok_pos, slots, inv_freq, head_dim, heads, q_out,
                                                               pages.args(), True, err, bias=bq)))))
        if ops.tc_gemm_qkv_takes(x, wq, head_dim):
            angles = ops.rope_table(tok_pos, inv_freq)
            print("  tcgen05 product with bias, rotation, cache write  " + rate_q(timed(lambda: ops.tc_gemm_qkv(
                x, wq, bq, angles, tok_seq, tok_pos, slots, heads, q_out, pages.args(), True, err))), flush=True)
        if int(err):
            raise RuntimeError(f"a kernel reported error word {int(err)}")


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="qwenforge_b200.measure", description=__doc__.split("\n\n")[0])
    p.add_argument("what", choices=["products", "chain", "phases", "attention", "decode-attention", "gemm"])
    p.add_argument("--preset", default="qwen2.5-0.5b")
    p.add_argument("--rows", default="8", type=lambda text: [int(v) for v in text.split(",")])
    p.add_argument("--repeat", type=int, default=12, help="layers, each with weights of its own, captured into one graph")
    p.add_argument("--tokens", default="2048", type=lambda text: [int(v) for v in text.split(",")])
    p.add_argument("--heads", type=int, default=14)
    p.add_argument("--kv-heads", type=int, default=2)
    p.add_argument("--head-dim", type=int, default=64)
    p.add_argument("--lengths", default="4000,4000,4000,4000,4000,4000,4000,4000", type=lambda text: [int(v) for v in text.split(",")],
                   help="decode-attention: the sequences' lengths")
    p.add_argument("--splits", type=int, default=8, help="decode-attention: the most runs of pages per sequence")
    args = p.parse_args(argv)
    ops.require_cuda("cuda", "the measurement")
    with torch.inference_mode():
        {"products": measure_products, "chain": measure_chain, "phases": measure_phases, "attention": measure_attention,
         "decode-attention": measure_decode_attention, "gemm": measure_gemm}[args.what](args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
