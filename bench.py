"""Measurement of qwenforge_b200 on one B200: decode tokens per second of a random-weight Qwen2.5-0.5B
(batch 8, context 4096 by default), with the prefill rate at 2,048 tokens, the decode step's HBM roofline,
decode at batch 1 and 64, and the same decode rate end to end through the Python entry point.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

One decode step = one token for every sequence of the batch. The K timed steps are the last K steps before
the context length is reached, so the cache is read at (almost) its full length. Timed with CUDA events on
the launching stream; the step's operands (about 1 GB of weights plus the cache) are far larger than the
126 MB L2, so no flush is needed between steps. Prints ONE JSON line.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=256)
    p.add_argument("--warmup", type=int, default=16)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--preset", default="qwen2.5-0.5b")
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--context", type=int, default=4096)
    p.add_argument("--prefill-tokens", type=int, default=2048)
    p.add_argument("--layers", type=int, default=None, help="run fewer layers than the preset has (both numbers are reported)")
    p.add_argument("--dtype", default="bfloat16")
    p.add_argument("--no-points", action="store_true", help="skip the batch 1 / batch 64 points and the end-to-end run")
    p.add_argument("--workload", default=None, choices=sorted(WORKLOADS),
                   help="run only this named workload (3B: 16 unequal prompts then 256 steps; 7B: batch 64 to context "
                        "8192 at temperature 0.7) and print its line")
    p.add_argument("--no-workloads", action="store_true", help="leave the 3B and 7B workloads out of the default run's points")
    return p.parse_args()


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return {"hbm_gbs": float(data.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"])),
                "bf16_tflops": float(data.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"])), "source": "measured"}
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs (read-only)."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.samples, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) == 6 and parts[0].isdigit():
                self.samples.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            self.proc.wait()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        mhz = sorted(int(s[0]) for s in self.samples)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": int(self.samples[0][1]), "reasons": reasons,
                "samples": len(mhz)}


def model_numbers(config, layers_run):
    """Bytes and FLOPs of one step from the configuration (bf16 weights, bf16 cache)."""
    h, i, d = config.hidden_size, config.intermediate_size, config.head_dim
    nh, kvh, v = config.num_attention_heads, config.num_key_value_heads, config.vocab_size
    per_layer = (nh + 2 * kvh) * d * h + (nh + 2 * kvh) * d + nh * d * h + 3 * i * h + 2 * h
    head = v * h
    weight_bytes = 2 * (layers_run * per_layer + head + h)
    kv_bytes_per_token = layers_run * 2 * kvh * d * 2
    linear_flops_per_token = 2 * layers_run * ((nh + 2 * kvh) * d * h + nh * d * h + 3 * i * h)
    return dict(weight_bytes=weight_bytes, kv_bytes_per_token=kv_bytes_per_token,
                linear_flops_per_token=linear_flops_per_token, head_flops_per_row=2 * head,
                attn_flops=lambda t: layers_run * 4 * nh * d * t * (t + 1) // 2)


def timed_decode(model, cache, batch, context, steps, warmup, vocab, torch):
    """Prefill `batch` prompts so that warmup + steps decode steps end at `context`, then replay the captured
    decode step (model, sampling, state update) from its CUDA graph. Returns (ms per timed step, kernels per step)."""
    from qwenforge_b200.engine.graphs import CHUNK_STEPS, DecodeGraph
    from qwenforge_b200.sampling import Sampler
    sampler = Sampler()
    prompt_len = context - steps - warmup
    g = torch.Generator().manual_seed(1234)
    slots = [cache.open() for _ in range(batch)]
    cache.reserve([(s, context) for s in slots])
    tokens = []
    for begin in range(0, batch, 8):  # prefill in chunks of 8 prompts to bound activation memory
        chunk = slots[begin:begin + 8]
        prompts = [torch.randint(0, vocab, (prompt_len,), generator=g).tolist() for _ in chunk]
        tokens += sampler(model.step(cache, list(zip(chunk, prompts)))).tolist()
    cache.flush()
    graph = DecodeGraph(model, cache, batch, context, sampler)
    graph.capture()
    graph.load(slots, tokens, [prompt_len] * batch, [1] * batch, [1 << 30] * batch, list(range(batch)), [])

    def run(n):
        for i in range(n):
            if i % CHUNK_STEPS == 0:
                graph.cursor.zero_()
            graph.graph.replay()

    run(warmup)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    run(steps)
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / steps
    model.raise_on_kernel_error()
    assert int(graph.tok_pos.max()) == context, "the timed steps did not end at the context length"
    for s in slots:
        cache.close(s)
    return ms, graph.kernels_per_step


def check_decode_logits(model, cache, folder, batch, context, vocab, torch, rows_checked=2):
    """Guards the number: 32 steps of the batch replayed from the decode graph that the timing used (same rows, same
    length bound), then the last step's bfloat16 logits of two rows against the logits that a float32 model of the
    same weights gives for the same tokens. Raises if they differ by more than the tests' bfloat16 tolerance."""
    from qwenforge_b200.engine import Model
    from qwenforge_b200.engine.graphs import CHUNK_STEPS, DecodeGraph
    from qwenforge_b200.sampling import Sampler
    sampler = Sampler()
    prompt_len = context - CHUNK_STEPS - 1
    g = torch.Generator().manual_seed(4321)
    slots = [cache.open() for _ in range(batch)]
    cache.reserve([(s, context) for s in slots])
    prompts, first = [], []
    for begin in range(0, batch, 8):
        chunk = slots[begin:begin + 8]
        part = [torch.randint(0, vocab, (prompt_len,), generator=g).tolist() for _ in chunk]
        prompts += part
        first += sampler(model.step(cache, list(zip(chunk, part)))).tolist()
    cache.flush()
    graph = DecodeGraph(model, cache, batch, context, sampler)
    graph.capture()
    graph.load(slots, first, [prompt_len] * batch, [1] * batch, [1 << 30] * batch, list(range(batch)), [])
    produced = graph.run(CHUNK_STEPS)
    got = graph.last_logits.float().cpu()
    model.raise_on_kernel_error()
    for s in slots:
        cache.close(s)
    exact = Model.from_dir(folder, "float32", "cuda:0")
    exact_cache = exact.new_cache(2 * (context + 64), 2)
    worst, bound, plain_worst, plain = 0.0, 0.0, None, None
    for row in sorted({0, batch - 1})[:rows_checked]:
        tokens = prompts[row] + [first[row]] + [step[row] for step in produced[:-1]]
        slot = exact_cache.open()
        ref = exact.step(exact_cache, [(slot, tokens)]).float().cpu()[0]
        exact_cache.close(slot)
        err = float((got[row] - ref).abs().max())
        limit = 2e-2 + 4e-2 * float(ref.abs().max())
        if err > limit:
            # The tests' tolerance is met by the default sizes; a deeper and wider model with random weights carries
            # more bfloat16 rounding to its logits whatever the kernels. Then the measure is the plain bfloat16 path
            # (the SIMT attention kernel, library products, no fusion) on the same tokens: the timed path may be no
            # further from float32 than that one, within a quarter.
            if plain is None:
                plain = Model.from_dir(folder, "bfloat16", "cuda:0", attention="generic")
            plain_cache = plain.new_cache(context + 64, 1)
            slot = plain_cache.open()
            plain_err = float((plain.step(plain_cache, [(slot, tokens)]).float().cpu()[0] - ref).abs().max())
            plain_cache.close(slot)
            del plain_cache
            if err > 1.25 * plain_err + 2e-2:
                raise AssertionError(f"decode graph logits of row {row} differ from float32 by {err:.3e} (limit {limit:.3e}; "
                                     f"the plain bfloat16 path differs by {plain_err:.3e})")
            plain_worst = max(plain_worst or 0.0, plain_err)
        worst, bound = max(worst, err), max(bound, limit)
    exact.raise_on_kernel_error()
    if plain is not None:
        plain.raise_on_kernel_error()
    del exact_cache, plain
    # the true 32-bit path's own speed, at a shorter context (its prompt step is slow): the same batch, graph replays
    short = min(context, 1024)
    exact_cache = exact.new_cache(batch * (short + 64), batch)
    fp32_ms, _ = timed_decode(exact, exact_cache, batch, short, 16, 3, vocab, torch)
    del exact, exact_cache
    torch.cuda.empty_cache()
    result = {"max_abs_diff_vs_fp32": round(worst, 5), "limit": round(bound, 5), "rows": rows_checked, "steps_replayed": CHUNK_STEPS,
              "fp32_decode_tokens_per_s": round(batch * 1e3 / fp32_ms, 1), "fp32_decode_ms_per_step": round(fp32_ms, 3),
              "fp32_decode_context": short}
    if plain_worst is not None:   # beyond the tests' tolerance, accepted against the plain bfloat16 path's own distance
        result["plain_bf16_diff_vs_fp32"] = round(plain_worst, 5)
    return result


# The two larger workloads: 16 prompts of unequal lengths in ONE prompt step, then 256 decode steps, at Qwen2.5-3B layer
# sizes; and batch 64 with 512-token prompts decoded to a context of 8,192 with temperature 0.7 at Qwen2.5-7B layer sizes.
WORKLOADS = {
    "3b": dict(preset="qwen2.5-3b", batch=16, prompt_range=(64, 2048), new_steps=256, temperature=0.0, seed=0),
    "7b": dict(preset="qwen2.5-7b", batch=64, prompt_range=(512, 512), context=8192, temperature=0.7, seed=0),
}


def run_workload(name, pk, torch, layers=None, timed_last=256):
    """One named workload with all of its layers (unless `layers` says otherwise), weights drawn on the device. All
    prompts run in ONE step, then every decode step is replayed from one CUDA graph; the decode rate is that of ALL
    the steps, and the last `timed_last` steps (the longest contexts) are also timed on their own."""
    from qwenforge_b200.config import preset_config
    from qwenforge_b200.engine import Model
    from qwenforge_b200.engine.graphs import CHUNK_STEPS, DecodeGraph
    from qwenforge_b200.sampling import Sampler, SamplingParams
    w = WORKLOADS[name]
    full = preset_config(w["preset"])
    layers_run = layers or full.num_hidden_layers
    config = preset_config(w["preset"], num_hidden_layers=layers_run)
    numbers = model_numbers(config, layers_run)
    batch = w["batch"]
    g = torch.Generator().manual_seed(99)
    lo, hi = w["prompt_range"]
    lengths = [int(torch.randint(lo, hi + 1, (1,), generator=g)) for _ in range(batch)]
    steps = w["new_steps"] if "new_steps" in w else w["context"] - max(lengths)
    model = Model.from_random(config, w["seed"], "bfloat16", "cuda:0")
    cache = model.new_cache(sum(-(-(n + steps) // 64) * 64 for n in lengths), batch, max(lengths) + steps)
    sampler = Sampler(SamplingParams(w["temperature"], w["seed"]))
    prompts = [torch.randint(0, config.vocab_size, (n,), generator=g).tolist() for n in lengths]
    ev = lambda: torch.cuda.Event(enable_timing=True)
    model.step(cache, [(-1, [1, 2, 3])], want=[[]])   # an untimed padding step: loads what a first step loads
    # The prompt step twice, launch by launch both times (no prompt graphs here): the process's first run of these
    # kernels at these sizes also loads them and lets the library choose its products; the second is what a step costs.
    prefill_runs = []
    for run in range(2):
        slots = [cache.open() for _ in range(batch)]
        cache.reserve([(s, n + steps) for s, n in zip(slots, lengths)])
        torch.cuda.synchronize()
        a, b = ev(), ev()
        a.record()
        logits = model.step(cache, list(zip(slots, prompts)))
        b.record()
        torch.cuda.synchronize()
        prefill_runs.append(a.elapsed_time(b))
        if run == 0:
            for s in slots:
                cache.close(s)
    prefill_ms = prefill_runs[1]
    seq_ids = torch.arange(batch, dtype=torch.int64, device="cuda:0")
    first = sampler(logits, seq_ids, torch.zeros(batch, dtype=torch.int32, device="cuda:0")).tolist()
    cache.flush()
    graph = DecodeGraph(model, cache, batch, max(lengths) + steps, sampler)
    graph.capture()
    graph.load(slots, first, lengths, [1] * batch, [1 << 30] * batch, list(range(batch)), [])
    timed_last = min(timed_last, steps)
    a, mid, b = ev(), ev(), ev()
    with ClockSampler() as clocks:
        a.record()
        for i in range(steps):
            if i % CHUNK_STEPS == 0:
                graph.cursor.zero_()
            if i == steps - timed_last:
                mid.record()
            graph.graph.replay()
        b.record()
        torch.cuda.synchronize()
    model.raise_on_kernel_error()
    assert int(graph.tok_pos.max()) == max(lengths) + steps, "the decode steps did not reach the planned length"
    ms_all, ms_last = a.elapsed_time(b) / steps, mid.elapsed_time(b) / timed_last
    total_tokens = sum(lengths)
    flops = numbers["linear_flops_per_token"] * total_tokens + numbers["head_flops_per_row"] * batch + sum(
        numbers["attn_flops"](n) for n in lengths)
    mean_len = sum(lengths) / batch
    bytes_all = numbers["weight_bytes"] + batch * (mean_len + steps / 2) * numbers["kv_bytes_per_token"]
    bytes_last = numbers["weight_bytes"] + batch * (mean_len + steps - timed_last / 2) * numbers["kv_bytes_per_token"]
    gbs_all, gbs_last = bytes_all / (ms_all * 1e-3) / 1e9, bytes_last / (ms_last * 1e-3) / 1e9
    out = {
        "workload": name, "model": w["preset"], "layers": layers_run, "layers_in_config": full.num_hidden_layers,
        "batch": batch, "prompt_tokens": total_tokens, "prompt_len_min": min(lengths), "prompt_len_max": max(lengths),
        "decode_steps": steps, "temperature": w["temperature"],
        "tokens_per_s": round(batch * 1e3 / ms_all, 1), "ms_per_step": round(ms_all, 4),
        "bytes_per_step": int(bytes_all), "gbs": round(gbs_all, 1), "roofline_frac": round(gbs_all / pk["hbm_gbs"], 4),
        "last_steps": timed_last, "last_ms_per_step": round(ms_last, 4), "last_tokens_per_s": round(batch * 1e3 / ms_last, 1),
        "last_roofline_frac": round(gbs_last / pk["hbm_gbs"], 4),
        "prefill_ms": round(prefill_ms, 3), "prefill_tokens_per_s": round(total_tokens / prefill_ms * 1e3, 1),
        "prefill_frac": round(flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
        "prefill_how": "ONE step of all prompts, launch by launch (its second run; the process's first run is prefill_first_ms)",
        "prefill_first_ms": round(prefill_runs[0], 3),
        "kernels_per_step": graph.kernels_per_step, "clocks": clocks.summary(),
    }
    for s in slots:
        cache.close(s)
    del graph, cache, model
    torch.cuda.empty_cache()
    return out


class _StubTokenizer:
    """Stands where the reference loads a tokenizer (there are no tokenizer files and no network): a prompt is the text
    "<length> <seed>" and encodes to that many seeded uniform-random token ids; ids decode to their decimal text."""
    pad_token_id, eos_token_id, bos_token_id = 0, 1, 1
    pad_token, eos_token, padding_side = "<pad>", "<eos>", "right"

    def __init__(self, vocab, torch):
        self.vocab, self.torch = vocab, torch

    def apply_chat_template(self, messages, tokenize=False, add_generation_prompt=True):
        return messages[0]["content"]

    def __call__(self, texts, add_special_tokens=False, padding=True, return_attention_mask=True, return_tensors="pt"):
        torch = self.torch
        rows = []
        for text in texts:
            length, seed = (int(x) for x in text.split())
            rows.append(torch.randint(2, self.vocab, (length,), generator=torch.Generator().manual_seed(seed)))
        longest = max(len(r) for r in rows)
        ids = torch.zeros(len(rows), longest, dtype=torch.long)
        mask = torch.zeros(len(rows), longest, dtype=torch.long)
        for i, r in enumerate(rows):
            ids[i, :len(r)] = r
            mask[i, :len(r)] = 1
        return {"input_ids": ids, "attention_mask": mask}

    def batch_decode(self, rows, skip_special_tokens=True, clean_up_tokenization_spaces=False):
        return [" ".join(str(t) for t in row) for row in rows]


def reference_arm(args):
    """The unmodified reference (a plain copy of its tree under baseline/_ref) through its own entry point,
    `StudentEngine(...).generate(prompts, max_new_tokens, batch_size)`, on the same random-weight model folder, batch,
    context and step count. Only its tokenizer loader is replaced by a stub (it is a script tree that pip cannot
    install, and its tokenizer files are not here). None of this library's kernels or models run: only the writer of
    the random-weight folder. The decode rate is the difference of two calls that share the prompt step: one that
    ends at the context length and one that stops `steps` tokens earlier."""
    import types
    unavailable = lambda why: print(json.dumps({"impl": "reference", "unavailable": why})) or 0
    ref_root = ROOT / "baseline" / "_ref"
    if not (ref_root / "student_engine.py").exists():
        return unavailable("baseline/_ref holds no copy of the reference tree (student_engine.py is missing)")
    if args.gpus != 1:
        return unavailable("the reference engine runs on one GPU")
    try:
        import torch
        if not torch.cuda.is_available():
            return unavailable("no CUDA device")
        sys.path.insert(0, str(ref_root))
        import student_engine as se
        from qwenforge_b200.config import preset_config
        from qwenforge_b200.weights import write_random_model
        config = preset_config(args.preset, num_hidden_layers=args.layers) if args.layers else preset_config(args.preset)
        layers_cfg = preset_config(args.preset).num_hidden_layers
        steps, warmup, batch, context = args.steps, max(args.warmup, 3), args.batch, args.context
        short_new = 9                       # the reference graphs runs of 8 or more new tokens (student_engine.py:1274)
        long_new = short_new + steps
        prompt_len = context - long_new + 1  # the long call's last token is fed at position context - 1
        with tempfile.TemporaryDirectory(prefix="qf_ref_") as folder:
            write_random_model(config, seed=0, out_dir=folder, store_dtype=torch.bfloat16)
            stub = _StubTokenizer(config.vocab_size, torch)
            se.AutoTokenizer = types.SimpleNamespace(from_pretrained=lambda *a, **k: stub)
            dtype = "float16"  # the reference's default; its own attention kernels are written for float16
            engine = se.StudentEngine(folder, device="cuda", dtype=dtype, attn_implementation="sdpa", local_files_only=True)
            prompts = [f"{prompt_len} {100 + i}" for i in range(batch)]

            def timed(new_tokens, texts=prompts, size=batch):
                torch.cuda.synchronize()
                start = time.perf_counter()
                out = engine.generate(texts, new_tokens, batch_size=size)
                torch.cuda.synchronize()
                assert len(out) == len(texts) and all(len(o.split()) == new_tokens for o in out)
                return (time.perf_counter() - start) * 1e3

            for _ in range(2):  # warm-up: compiles its pointwise kernels, captures both decode graphs
                timed(short_new)
                timed(long_new)
            repeats = 1 + max(1, warmup // 3)
            with ClockSampler() as clocks:
                shorts = sorted(timed(short_new) for _ in range(repeats))
                longs = sorted(timed(long_new) for _ in range(repeats))
            ms = (longs[len(longs) // 2] - shorts[len(shorts) // 2]) / steps
            value = batch * 1e3 / ms
            ttft = sorted(timed(1, [f"{args.prefill_tokens} 7"], 1) for _ in range(5))[2:]
            prefill_ms = ttft[len(ttft) // 2]
            graphs = bool(getattr(engine, "_graph_decode_enabled", False)) and bool(getattr(engine, "_graph_ctx", None))
        line = {
            "impl": "reference", "metric": "decode tokens/s (batch %d, context %d)" % (batch, context),
            "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
            "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "fp16", "data": "synthetic (seeded uniform-random token ids, seeded random weights)",
            "config": {"model": args.preset, "layers": config.num_hidden_layers, "layers_in_config": layers_cfg,
                       "global_batch": batch, "seq_len": context, "prefill_tokens": args.prefill_tokens,
                       "parallelism": "single GPU", "decode_graphs": graphs,
                       "timing": "host clock around generate(); decode = (call ending at the context - call ending "
                                 "%d tokens earlier) / %d" % (steps, steps)},
            "clocks": clocks.summary(),
            "prefill": {"value": round(args.prefill_tokens / prefill_ms * 1e3, 1), "tokens": args.prefill_tokens,
                        "ms": round(prefill_ms, 3), "note": "generate() of one prompt with max_new_tokens=1"},
            "e2e": {"value": round(value, 1), "unit": "tokens/s",
                    "note": "the same figure: every call goes through StudentEngine.generate, strings in and out"},
            "call_ms": {"short": round(shorts[len(shorts) // 2], 2), "long": round(longs[len(longs) // 2], 2)},
        }
        print(json.dumps(line))
        return 0
    except Exception as exc:  # the reference could not be driven here: say why, in one line
        return unavailable(f"{type(exc).__name__}: {str(exc).splitlines()[0] if str(exc) else ''}"[:300])


def main():
    args = parse()
    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print("bench.py: this library runs on ONE GPU; --gpus N > 1 is not supported")
        return 2

    import torch

    from qwenforge_b200.config import preset_config
    from qwenforge_b200.engine import Model, StudentEngine
    from qwenforge_b200.weights import write_random_model

    pk = peaks()
    if args.workload:
        with torch.inference_mode():
            out = run_workload(args.workload, pk, torch, args.layers)
        line = {"metric": "decode tokens/s (%s workload: batch %d, %d steps)" % (args.workload, out["batch"], out["decode_steps"]),
                "value": out["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": out["decode_steps"], "warmup": 0,
                "ms_per_step": out["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "bf16", "data": "synthetic (seeded uniform-random token ids, weights drawn on the device)",
                "config": {k: out[k] for k in ("model", "layers", "layers_in_config", "batch", "prompt_tokens",
                                               "prompt_len_min", "prompt_len_max", "decode_steps", "temperature")},
                "clocks": out.pop("clocks"), "gpu_launches": out["kernels_per_step"] * out["decode_steps"],
                "roofline": {"bound": "hbm", "achieved": out["gbs"], "peak": pk["hbm_gbs"], "unit": "GB/s",
                             "frac": out["roofline_frac"], "peaks": pk["source"]},
                "prefill": {"value": out["prefill_tokens_per_s"], "tokens": out["prompt_tokens"], "ms": out["prefill_ms"],
                            "frac": out["prefill_frac"], "first_ms": out["prefill_first_ms"], "how": out["prefill_how"]},
                "workload": out}
        print(json.dumps(line))
        return 0
    full = preset_config(args.preset)
    layers_cfg = full.num_hidden_layers
    layers_run = args.layers or layers_cfg
    config = preset_config(args.preset, num_hidden_layers=layers_run)
    numbers = model_numbers(config, layers_run)
    steps, warmup, batch, context = args.steps, max(args.warmup, 3), args.batch, args.context

    with tempfile.TemporaryDirectory(prefix="qf_bench_") as folder, torch.inference_mode():
        write_random_model(config, seed=0, out_dir=folder, store_dtype=torch.bfloat16)
        model = Model.from_dir(folder, args.dtype, "cuda:0")
        model.enable_prefill_graphs()  # as StudentEngine does: a prompt shape that comes back is replayed from a graph
        vocab = config.vocab_size
        cache = model.new_cache(max(batch, 64 if not args.no_points else batch) * context, 64)

        # ---- prefill of 2,048 tokens, one sequence
        g = torch.Generator().manual_seed(7)
        prompt = torch.randint(0, vocab, (args.prefill_tokens,), generator=g).tolist()
        times = []
        for rep in range(5):
            slot = cache.open()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            model.step(cache, [(slot, prompt)])
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
            cache.close(slot)
        prefill_ms = sorted(times[2:])[len(times[2:]) // 2]
        # the same prompt as a shape that was not seen before (another number of wanted rows): issued launch by launch
        firsts = []
        for extra in (2, 3, 4):
            slot = cache.open()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            model.step(cache, [(slot, prompt)], want=[list(range(args.prefill_tokens - extra, args.prefill_tokens))])
            b.record()
            torch.cuda.synchronize()
            firsts.append(a.elapsed_time(b))
            cache.close(slot)
        first_ms = sorted(firsts)[1]
        # prompts of lengths that never came before, a few tokens short of the prompt above: the first two bring their
        # rounded shape (a padding entry fills every one up to the same token count) and capture it, the others replay it
        news = []
        for short in (5, 17, 29, 41, 53):
            slot = cache.open()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            model.step(cache, [(slot, prompt[:args.prefill_tokens - short])])
            b.record()
            torch.cuda.synchronize()
            news.append(a.elapsed_time(b))
            cache.close(slot)
        new_ms = sorted(news[2:])[1]
        t = args.prefill_tokens
        prefill_flops = numbers["linear_flops_per_token"] * t + numbers["attn_flops"](t) + numbers["head_flops_per_row"]
        frac = lambda ms: round(prefill_flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)
        prefill = {"value": round(t / prefill_ms * 1e3, 1), "tokens": t, "ms": round(prefill_ms, 3), "frac": frac(prefill_ms),
                   "how": "a prompt shape that came before, replayed from its CUDA graph (median of 3)",
                   "first_seen_ms": round(first_ms, 3), "first_seen_frac": frac(first_ms),
                   "first_seen_value": round(t / first_ms * 1e3, 1),
                   "new_length_ms": round(new_ms, 3)}   # a length never seen, in a rounded shape that was (about 2,010 tokens)

        # ---- the headline: decode at the default batch, with clocks sampled meanwhile
        with ClockSampler() as clocks:
            ms, per_step = timed_decode(model, cache, batch, context, steps, warmup, vocab, torch)
        gpu_launches = per_step * steps  # this library's own kernels in the timed replays (library GEMMs not counted)
        value = batch * 1e3 / ms
        mean_ctx = context - steps / 2
        step_bytes = numbers["weight_bytes"] + batch * mean_ctx * numbers["kv_bytes_per_token"]
        achieved = step_bytes / (ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                    "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk["source"]}

        # ---- the timed path gives the right logits: a step replayed from the same decode graph against float32
        logits_check = check_decode_logits(model, cache, folder, batch, context, vocab, torch)

        points, e2e = {}, None
        if not args.no_points:
            for b in (1, 64):
                k = min(steps, 128)
                points[f"decode_b{b}"] = round(b * 1e3 / timed_decode(model, cache, b, context, k, 4, vocab, torch)[0], 1)
            # ---- end to end through the entry point: host token ids in, host token ids out, every step
            del cache
            engine = StudentEngine(folder, device="cuda:0", dtype=args.dtype)
            k = min(steps, 128)
            prompts = [torch.randint(0, vocab, (context - k - 1,), generator=g).tolist() for _ in range(batch)]
            engine.generate_ids(prompts, 9, batch_size=batch, ignore_eos=True)  # warm-up: compiles nothing new, captures the graph
            engine.generate_ids(prompts, k + 1, batch_size=batch, ignore_eos=True)  # one untimed run of the same call
            engine.generate_ids(prompts, k + 1, batch_size=batch, ignore_eos=True)
            loop = engine.last_loop
            # copies of the decode phase, from the tensors copied: the rows' state once per batch of requests
            # (5 int32 + 1 int64 per row, 8 stop ids), the produced tokens and the error word once per chunk of steps
            chunks = -(-loop.steps_run // 32)
            e2e = {"value": round(loop.decoded_tokens / loop.decode_seconds, 1), "unit": "tokens/s",
                   "h2d_bytes_per_step": round((28 * batch + 32) / max(loop.steps_run, 1), 2),
                   "d2h_bytes_per_step": round(chunks * (4 * 32 * batch + 4) / max(loop.steps_run, 1), 2),
                   "note": "StudentEngine.generate_ids: host token ids in, host token ids out; decode replays CUDA "
                           "graphs and reads tokens back every 32 steps"}

    if not args.no_points and not args.no_workloads and args.layers is None:
        with torch.inference_mode():
            for name in sorted(WORKLOADS):
                out = run_workload(name, pk, torch)
                for key in ("tokens_per_s", "ms_per_step", "roofline_frac", "last_ms_per_step", "last_roofline_frac",
                            "prefill_ms", "prefill_frac"):
                    points[f"w{name}_{key}"] = out[key]

    line = {
        "metric": "decode tokens/s (batch %d, context %d)" % (batch, context), "value": round(value, 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if args.dtype.startswith("bf") else "fp32",
        "data": "synthetic (seeded uniform-random token ids, seeded random weights)",
        "config": {"model": args.preset, "layers": layers_run, "layers_in_config": layers_cfg,
                   "hidden": config.hidden_size, "heads": config.num_attention_heads,
                   "kv_heads": config.num_key_value_heads, "head_dim": config.head_dim,
                   "intermediate": config.intermediate_size, "vocab": config.vocab_size,
                   "global_batch": batch, "seq_len": context, "prefill_tokens": args.prefill_tokens,
                   "parallelism": "single GPU", "l2": "operands larger than L2 (weights ~1 GB per step); no flush",
                   "tied_head": config.tie_word_embeddings},
        "clocks": clocks.summary(), "gpu_launches": gpu_launches, "prefill": prefill, "roofline": roofline,
        "points": points, "e2e": e2e, "logits_check": logits_check,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
