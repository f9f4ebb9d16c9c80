"""bin/trace_run as a user runs it: a subprocess, JSON steps on standard input, logits files out. The same requests
are replayed whole, with the last 32 tokens one by one, and in unequal batches whose requests end at different steps."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tests import plain_qwen2 as plain
from tests.helpers import TINY_A, TINY_B, TINY_W, assert_logits_close, make_model_dir, random_tokens

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def run_trace(model_dir, dtype, steps, out_dir, max_tokens):
    text = "".join(json.dumps(s) + "\n" for s in steps)
    done = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
                           "--out", str(out_dir), "--max-tokens", str(max_tokens)],
                          input=text, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [line for line in done.stdout.splitlines() if line.startswith("done ")] == [f"done {s['step']}" for s in steps]
    return done


def read(out_dir, step, vocab):
    data = np.fromfile(Path(out_dir) / f"{step}.f32", dtype="<f4")
    return torch.from_numpy(data.reshape(-1, vocab).copy())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("config", [TINY_A, TINY_B, TINY_W], ids=["tiny_a", "tiny_b", "tiny_w"])
def test_three_ways_of_cutting(config, dtype, tmp_path):
    folder, weights = make_model_dir(config, 2, tmp_path / "model")
    vocab = config["vocab_size"]
    torch_dtype = torch.float32 if dtype == "float32" else torch.bfloat16
    requests = {f"r{i}": random_tokens(vocab, n, 50 + i) for i, n in enumerate((40, 97, 130, 64, 33))}
    refs = {k: plain.forward_logits(config, weights, v) for k, v in requests.items()}

    # 1. each request alone and whole
    steps = [dict(step=i, entries=[dict(id=k, tokens=v, want=list(range(len(v))))], end=[k])
             for i, (k, v) in enumerate(requests.items())]
    run_trace(folder, dtype, steps, tmp_path / "whole", max_tokens=192)
    for i, k in enumerate(requests):
        assert_logits_close(read(tmp_path / "whole", i, vocab), refs[k], torch_dtype, f"whole {k}")

    # 2. all but the last 32 tokens in one step, then one by one; a step that wants nothing writes no file
    k, v = "r2", requests["r2"]
    head = len(v) - 32
    steps = [dict(step=0, entries=[dict(id=k, tokens=v[:head], want=[])], end=[])]
    steps += [dict(step=1 + t, entries=[dict(id=k, tokens=[v[head + t]], want=[0])], end=[k] if t == 31 else [])
              for t in range(32)]
    run_trace(folder, dtype, steps, tmp_path / "tail", max_tokens=192)
    assert not (tmp_path / "tail" / "0.f32").exists()
    tail = torch.cat([read(tmp_path / "tail", 1 + t, vocab) for t in range(32)])
    assert_logits_close(tail, refs[k][head:], torch_dtype, "last 32 one by one")

    # 3. two batches of unequal lengths, one after the other, in a cache too small for both: prompts minus 8 tokens
    #    start together, then one token each; shorter requests end earlier
    steps, n = [], 0
    collected = {k: [] for k in requests}
    plan = []
    for batch in (["r0", "r1", "r2"], ["r3", "r4", "r1"]):
        heads = {k: len(requests[k]) - 8 - (3 if k == "r0" else 0) for k in batch}
        steps.append(dict(step=n, entries=[dict(id=f"{k}@{n}", tokens=requests[k][:heads[k]], want=list(range(heads[k])))
                                           for k in batch], end=[]))
        plan.append((n, [(k, heads[k]) for k in batch]))
        first = n
        n += 1
        fed = dict(heads)
        while any(fed[k] < len(requests[k]) for k in batch):
            live = [k for k in batch if fed[k] < len(requests[k])]
            entries = [dict(id=f"{k}@{first}", tokens=[requests[k][fed[k]]], want=[0]) for k in live]
            for k in live:
                fed[k] += 1
            steps.append(dict(step=n, entries=entries, end=[f"{k}@{first}" for k in live if fed[k] == len(requests[k])]))
            plan.append((n, [(k, 1) for k in live]))
            n += 1
    run_trace(folder, dtype, steps, tmp_path / "batches", max_tokens=64 * 6)
    for step, parts in plan:
        data = read(tmp_path / "batches", step, vocab)
        o = 0
        for k, count in parts:
            collected[k].append(data[o:o + count])
            o += count
        assert o == data.shape[0]
    for k in requests:
        got = torch.cat(collected[k])
        want = torch.cat([refs[k]] * (got.shape[0] // refs[k].shape[0]))
        assert_logits_close(got, want, torch_dtype, f"batched {k}")


def test_too_small_a_cache_fails_loudly(tmp_path):
    folder, _ = make_model_dir(TINY_A, 2, tmp_path / "model")
    text = json.dumps(dict(step=0, entries=[dict(id="a", tokens=list(range(70)), want=[0])], end=[])) + "\n"
    done = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32",
                           "--out", str(tmp_path / "o"), "--max-tokens", "64"], input=text, capture_output=True,
                          text=True, timeout=600)
    assert done.returncode != 0 and "CacheFull" in done.stderr


def test_command_line_runs_a_small_suite(tmp_path):
    done = subprocess.run([sys.executable, "-m", "qwenforge_b200.cli", "--random-weights", "tiny-b", "--dtype", "bfloat16",
                           "--suites", "decode_throughput,ttft_prefill", "--decode-batch-sizes", "1,3",
                           "--decode-prompt-lens", "5,9,17", "--ttft-prompt-lens", "33,64", "--max-new-tokens-decode", "12",
                           "--timed-repeats", "2", "--output-dir", str(tmp_path / "out")],
                          capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert done.returncode == 0, done.stderr[-2000:]
    summary = json.loads((tmp_path / "out" / "summary.json").read_text())
    rows = summary["results"]
    assert [r["suite"] for r in rows] == ["decode_throughput", "decode_throughput", "ttft_prefill"]
    assert rows[1]["batch_size"] == 3 and rows[1]["new_tokens"] == 3 * 12 and all(r["tokens_per_s"] > 0 for r in rows)


def test_command_line_context_length_range_and_kernel_times(tmp_path):
    peaks = tmp_path / "peaks.json"
    peaks.write_text(json.dumps({"hbm_gbs": 6500.0}))
    done = subprocess.run([sys.executable, "-m", "qwenforge_b200.cli", "--random-weights", "tiny-a", "--dtype", "bfloat16",
                           "--suites", "decode_throughput", "--decode-batch-sizes", "4", "--prompt-len-range", "5,30",
                           "--context", "48", "--time-kernels", "--peaks", str(peaks), "--output-dir", str(tmp_path / "out")],
                          capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert done.returncode == 0, done.stderr[-2000:]
    summary = json.loads((tmp_path / "out" / "summary.json").read_text())
    row = summary["results"][0]
    assert row["requests"] == 4 and 4 * (48 - 30) <= row["new_tokens"] <= 4 * (48 - 5)   # every request decoded to 48 tokens
    assert row["bytes_per_step"] > 0 and row["decode_gbs"] > 0 and 0 < row["decode_roofline_frac"] < 1
    assert row["peak_memory_bytes"] > 0
    kernels = {k["kernel"] for k in summary["kernels"]}
    assert any(k.startswith("linear[") for k in kernels) and "embed_gather" in kernels and "sample" in kernels
    assert "kernel" in done.stdout and "us/call" in done.stdout


def test_validate_program(tmp_path):
    done = subprocess.run([sys.executable, "-m", "qwenforge_b200.validate", "--random-weights", "tiny-b", "--dtype", "float32"],
                          capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert done.returncode == 0, done.stderr[-2000:]
    assert "Signature check passed." in done.stdout and "Runtime interface check passed." in done.stdout


def test_dump_layers_of_trace_run(tmp_path):
    folder, weights = make_model_dir(TINY_B, 2, tmp_path / "model")
    tokens = random_tokens(TINY_B["vocab_size"], 9, 5)
    text = json.dumps(dict(step=0, entries=[dict(id="a", tokens=tokens, want=[8])], end=["a"])) + "\n"
    done = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32",
                           "--out", str(tmp_path / "o"), "--max-tokens", "64", "--dump-layers", str(tmp_path / "layers")],
                          input=text, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    sizes = plain.read_sizes(TINY_B)
    w64 = {k: v.double() for k, v in weights.items()}
    h = w64["model.embed_tokens.weight"][torch.tensor(tokens)]
    cos, sin = plain.rope_cos_sin(torch.arange(len(tokens)), sizes["head_dim"], sizes["theta"], torch.float64)
    for k in range(sizes["layers"] + 1):
        data = np.fromfile(tmp_path / "layers" / f"0.layer{k}.f32", dtype="<f4").reshape(len(tokens), -1)
        assert float((torch.from_numpy(data.copy()).double() - h).abs().max()) <= 2e-5 * max(1.0, float(h.abs().max()))
        if k < sizes["layers"]:
            h = plain.decoder_layer(h, w64, k, sizes, cos, sin)
