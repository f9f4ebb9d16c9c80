"""Trace replay: feed given token ids through a model step by step and write logits. Nothing is sampled.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps come on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

`entries` gives each request's next tokens and the places among them whose logits are wanted; `end`
names requests that are finished after the step (their cache slot and pages are given back). For a step
that wants something, `<out>/<step>.f32` receives the logits at the wanted places, in the order of the
entries and of `want`, as little-endian float32 [wanted, vocab]. After every step `done <step>` is
printed and flushed. `--max-tokens` is the most tokens live requests hold at any time, each request's
count rounded up to the cache's page of 64; it sizes the cache.

`--dump-layers DIR` also writes, for every step, the residual stream of the step's tokens after the embedding
(`DIR/<step>.layer0.f32`) and after every schedule entry k (`DIR/<step>.layer<k+1>.f32`), float32 [tokens, width]:
with `--dtype float32` an ordered trace to lay beside a plain implementation's when logits differ, in the manner
of the reference's whiteboard model (whiteboard_minimal_transformer/whiteboard_llm_inference.py:465-487).

This program has no forward pass, cache or loader of its own: it drives `Model.from_dir`,
`Model.new_cache` and `Model.step`, the ones generation uses.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

from ..cache import PAGE_TOKENS, round_up
from .model import Model


def parse_args(argv=None):
    p = argparse.ArgumentParser(prog="trace_run", description="Replay a token trace and write logits.")
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    p.add_argument("--out", required=True, help="folder that receives <step>.f32")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="most tokens live requests hold at any time (each rounded up to 64)")
    p.add_argument("--dump-layers", default=None, metavar="DIR",
                   help="also write the residual stream after the embedding and after every schedule entry")
    p.add_argument("--device", default="cuda")
    p.add_argument("--attn-implementation", default="sdpa",
                   help="'sdpa': fastest attention kernels that take the shapes; anything else: the plain SIMT kernel")
    return p.parse_args(argv)


def replay(model: Model, cache, lines, out_dir: Path, report=print, dump_dir: Path | None = None) -> None:
    slots: dict[str, int] = {}
    current = {"step": None}
    if dump_dir is not None:
        def observe(index, hidden, delta):
            stream = hidden if delta is None else hidden + delta.to(torch.float32)
            stream.cpu().contiguous().numpy().astype("<f4", copy=False).tofile(dump_dir / f"{current['step']}.layer{index}.f32")
        model.observer = observe
    for line in lines:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = current["step"] = record["step"]
        entries, want = [], []
        for item in record.get("entries", []):
            key = str(item["id"])
            if key not in slots:
                slots[key] = cache.open()
            entries.append((slots[key], [int(t) for t in item["tokens"]]))
            want.append([int(w) for w in item.get("want", [])])
        if entries:
            logits = model.step(cache, entries, want)
            if logits is not None:
                data = logits.to(torch.float32).cpu().contiguous().numpy().astype("<f4", copy=False)
                data.tofile(out_dir / f"{step}.f32")
            model.raise_on_kernel_error()
        for key in record.get("end", []):
            key = str(key)
            if key in slots:
                cache.close(slots.pop(key))
        report(f"done {step}")


def main(argv=None) -> int:
    args = parse_args(argv)
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    attention = "auto" if args.attn_implementation.lower() in ("sdpa", "flash", "auto") else "generic"
    with torch.inference_mode():
        model = Model.from_dir(args.model, args.dtype, args.device, attention)
        n_tokens = round_up(max(args.max_tokens, 1), PAGE_TOKENS)
        cache = model.new_cache(n_tokens, max_seqs=min(n_tokens // PAGE_TOKENS, 4096))
        dump_dir = Path(args.dump_layers) if args.dump_layers else None
        if dump_dir is not None:
            dump_dir.mkdir(parents=True, exist_ok=True)
        replay(model, cache, sys.stdin, out_dir, report=lambda text: print(text, flush=True), dump_dir=dump_dir)
    return 0


if __name__ == "__main__":
    sys.exit(main())
