"""Command line of qwenforge_b200, in the manner of the reference's scripts/run_inference_benchmark.py:88-153.

    python -m qwenforge_b200.cli --model DIR [--dtype bfloat16] [--suites decode_throughput,ttft_prefill] ...
    python -m qwenforge_b200.cli --random-weights qwen2.5-0.5b --suites decode_throughput --decode-batch-sizes 1,8
    python -m qwenforge_b200.cli --model DIR --prompt "some text" --max-new-tokens-decode 32

Options that the reference has keep its names and meanings: --model, --device, --dtype, --attn-implementation,
--local-files-only, --seed, --suites, --output-dir, --limit, --decode-batch-sizes, --ttft-batch-sizes,
--max-new-tokens-decode, --max-new-tokens-ttft, --warmup-iters (global warm-up generate calls), --batch-warmup-iters
(untimed calls per batch), --timed-repeats (timed calls per batch; the median is kept), --verbose-batches.
The reference's text workloads and its scoring against a saved baseline are not part of this library: the suites
here run on seeded random token ids of the lengths given by --decode-prompt-lens / --ttft-prompt-lens (defaults are
the lengths of the reference's published runs). Added: --random-weights PRESET (writes a seeded random model to a
temporary folder), --temperature, --stop-token-ids, --ignore-eos, --no-graphs, --prompt; --context N (each request of
the decode suite decodes until it holds N tokens) and --prompt-len-range LO,HI (its prompt lengths are drawn uniformly
from the range, one per request: an unequal batch); --time-kernels (device time of every kernel call, by CUDA events;
steps are then issued launch by launch); --peaks FILE (JSON with hbm_gbs: decode rows then carry their fraction of it).
Every row reports, beside latency and tokens per second, the bytes a decode step reads (weights once, the live
sequences' keys and values), the rate at which the decode phase read them, and the peak device memory.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import tempfile
import time
from pathlib import Path

ALL_SUITES = ("decode_throughput", "ttft_prefill")


def parse_args(argv=None) -> argparse.Namespace:
    p = argparse.ArgumentParser(prog="qwenforge_b200", description=__doc__.split("\n\n")[0])
    p.add_argument("--model", default=os.environ.get("HF_MODEL_NAME"), help="model folder (or hub id found in the local cache)")
    p.add_argument("--random-weights", metavar="PRESET", default=None,
                   help="use a seeded random model of a named size instead of --model (see config/presets)")
    p.add_argument("--device", default=os.environ.get("HF_DEVICE", "cuda"))
    p.add_argument("--dtype", choices=["auto", "float16", "bfloat16", "float32"], default="bfloat16",
                   help="float16 (the reference's default) is served by the bfloat16 path")
    p.add_argument("--attn-implementation", default="sdpa",
                   help="'sdpa': the fastest attention kernels that take the shapes; anything else: the plain SIMT kernel")
    p.add_argument("--local-files-only", action="store_true")
    p.add_argument("--seed", type=int, default=0, help="weights (random mode), token ids and sampling")
    p.add_argument("--suites", default=",".join(ALL_SUITES))
    p.add_argument("--output-dir", default=None)
    p.add_argument("--limit", type=int, default=None, help="first N cases of each suite")
    p.add_argument("--decode-batch-sizes", default="1,2,4")
    p.add_argument("--ttft-batch-sizes", default="1")
    p.add_argument("--max-new-tokens-decode", type=int, default=128)
    p.add_argument("--max-new-tokens-ttft", type=int, default=1)
    p.add_argument("--decode-prompt-lens", default="183,212,245,275", help="prompt lengths of the decode suite")
    p.add_argument("--ttft-prompt-lens", default="171,246,1000,1031,2175,3152,4719,7069")
    p.add_argument("--context", type=int, default=None,
                   help="decode suite: every request generates until its sequence holds this many tokens")
    p.add_argument("--prompt-len-range", default=None, metavar="LO,HI",
                   help="decode suite: prompt lengths drawn uniformly from [LO, HI], one per request of a batch")
    p.add_argument("--time-kernels", action="store_true",
                   help="print the device time of every kernel call (CUDA events; implies --no-graphs)")
    p.add_argument("--peaks", default=None, metavar="FILE", help="JSON file with hbm_gbs, the bandwidth the fractions are of")
    p.add_argument("--warmup-iters", type=int, default=1)
    p.add_argument("--batch-warmup-iters", type=int, default=0)
    p.add_argument("--timed-repeats", type=int, default=1)
    p.add_argument("--verbose-batches", action="store_true")
    p.add_argument("--temperature", type=float, default=0.0, help="0 = greedy")
    p.add_argument("--stop-token-ids", default="", help="comma list; default: the model's eos token")
    p.add_argument("--ignore-eos", action="store_true", help="always generate the full budget, as the reference does")
    p.add_argument("--no-graphs", action="store_true", help="decode step by step instead of replaying CUDA graphs")
    p.add_argument("--own-gemm", action="store_true",
                   help="run the projections of steps with 128 or more tokens on the library's own tcgen05 kernel "
                        "instead of cuBLAS (slower at present; see ops/linear.py)")
    p.add_argument("--prompt", action="append", default=None, help="generate text for this prompt (repeatable) and exit")
    args = p.parse_args(argv)
    if not args.model and not args.random_weights:
        p.error("give --model DIR or --random-weights PRESET")
    return args


def _ints(text: str) -> list:
    return [int(x) for x in str(text).split(",") if x.strip()]


def run_suite(engine, name, prompt_lens, batch_sizes, max_new, args, vocab, peaks=None) -> list:
    import torch
    rows = []
    g = torch.Generator().manual_seed(args.seed + 1)
    lens = prompt_lens[:args.limit] if args.limit else prompt_lens
    stops = _ints(args.stop_token_ids) or None
    decode_suite = name == "decode_throughput"
    for batch in batch_sizes:
        if decode_suite and args.prompt_len_range:
            lo, hi = _ints(args.prompt_len_range)
            sizes = [int(torch.randint(lo, hi + 1, (1,), generator=g)) for _ in range(batch)]
        else:
            sizes = [lens[i % len(lens)] for i in range(max(batch, len(lens)))]
        prompts = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in sizes]
        budgets = [max(args.context - n, 1) for n in sizes] if decode_suite and args.context else max_new
        kw = dict(batch_size=batch, temperature=args.temperature, seed=args.seed, stop_token_ids=stops,
                  ignore_eos=args.ignore_eos or stops is None)
        for _ in range(args.batch_warmup_iters):
            engine.generate_ids(prompts, budgets, **kw)
        times, tokens = [], 0
        torch.cuda.reset_peak_memory_stats()
        for _ in range(max(args.timed_repeats, 1)):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            out = engine.generate_ids(prompts, budgets, **kw)
            torch.cuda.synchronize()
            times.append(time.perf_counter() - t0)
            tokens = sum(len(t) for t in out)
        latency = statistics.median(times)
        loop = engine.last_loop
        row = dict(suite=name, batch_size=batch, requests=len(prompts), prompt_tokens=sum(len(p) for p in prompts),
                   new_tokens=tokens, latency_s=round(latency, 6), tokens_per_s=round(tokens / latency, 2),
                   decode_tokens_per_s=round(loop.decoded_tokens / loop.decode_seconds, 2) if loop.decode_seconds > 0 else None,
                   peak_memory_bytes=int(torch.cuda.max_memory_allocated()))
        if loop.steps_run and loop.decode_seconds > 0:
            # what a decode step of this run read on average: every weight once, and the keys and values of the
            # sequences that were live (each at the middle of its generation)
            live = loop.decoded_tokens / loop.steps_run
            middle = [len(p) + len(t) / 2 for p, t in zip(prompts, out)]
            step_bytes = engine.model.step_weight_bytes() + engine.cache.read_bytes(middle) * live / len(prompts)
            gbs = step_bytes * loop.steps_run / loop.decode_seconds / 1e9
            row.update(decode_steps=loop.steps_run, bytes_per_step=int(step_bytes), decode_gbs=round(gbs, 3))
            if peaks and peaks.get("hbm_gbs"):
                row["decode_roofline_frac"] = round(gbs / float(peaks["hbm_gbs"]), 6)
        rows.append(row)
        if args.verbose_batches or not args.output_dir:
            print(json.dumps(row), flush=True)
    return rows


def main(argv=None) -> int:
    args = parse_args(argv)
    import torch

    from .config import preset_config
    from .engine import StudentEngine
    from .weights import write_random_model

    if args.own_gemm:
        from .ops import use_own_tensor_core_products
        use_own_tensor_core_products(True)
    holder = None
    model_path = args.model
    if args.random_weights:
        holder = tempfile.TemporaryDirectory(prefix="qf_random_")
        model_path = holder.name
        store = torch.float32 if args.dtype == "float32" else torch.bfloat16
        write_random_model(preset_config(args.random_weights), args.seed, model_path, store)
    try:
        engine = StudentEngine(model_path, device=args.device, dtype=args.dtype,
                               attn_implementation=args.attn_implementation, local_files_only=args.local_files_only,
                               seed=args.seed, cuda_graphs=not (args.no_graphs or args.time_kernels))
        peaks = json.loads(Path(args.peaks).read_text()) if args.peaks else None
        if args.prompt:
            for text in engine.generate(list(args.prompt), args.max_new_tokens_decode, batch_size=len(args.prompt)):
                print(text)
            return 0
        vocab = engine.model.spec.vocab_size
        for _ in range(args.warmup_iters):
            engine.generate_ids([[1, 2, 3]], 8, ignore_eos=True)
        results = []
        suites = [s for s in args.suites.split(",") if s.strip()]
        timer = None
        if args.time_kernels:
            from .ops.timing import KernelTimer
            timer = KernelTimer().__enter__()
        try:
            for suite in suites:
                if suite == "decode_throughput":
                    results += run_suite(engine, suite, _ints(args.decode_prompt_lens), _ints(args.decode_batch_sizes),
                                         args.max_new_tokens_decode, args, vocab, peaks)
                elif suite == "ttft_prefill":
                    results += run_suite(engine, suite, _ints(args.ttft_prompt_lens), _ints(args.ttft_batch_sizes),
                                         args.max_new_tokens_ttft, args, vocab, peaks)
                else:
                    raise SystemExit(f"unknown suite {suite!r}; known: {', '.join(ALL_SUITES)}")
        finally:
            if timer is not None:
                timer.__exit__(None, None, None)
                print(timer.report(), flush=True)
        if args.output_dir:
            out = Path(args.output_dir)
            out.mkdir(parents=True, exist_ok=True)
            summary = dict(model=str(args.model or args.random_weights), dtype=args.dtype, seed=args.seed, results=results)
            if timer is not None:
                summary["kernels"] = [dict(kernel=k, calls=c, total_ms=round(ms, 4)) for k, c, ms in timer.totals()]
            (out / "summary.json").write_text(json.dumps(summary, indent=1))
        return 0
    finally:
        if holder is not None:
            holder.cleanup()


if __name__ == "__main__":
    sys.exit(main())
