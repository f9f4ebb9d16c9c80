"""Makes `reference_outputs.json`: logits of the reference's own engine on two tiny random models.

Run once, on the CPU, from the repository root with the reference checkout's path:

    python tests/golden/make_reference_outputs.py /path/to/QwenForge

It imports the reference's `student_engine.py` unchanged, replaces only its tokenizer loader with a stub
(the engine is driven with token ids, never with text), builds `StudentEngine(dir, device="cpu",
dtype="float32", attn_implementation="eager")` on model folders written from the tests' own random weights
(`tests/plain_qwen2.random_weights`, seeds below) and records, for every prompt (at 24 evenly spaced vocabulary columns, plus the row's maximum and the
greedy token): the last-position logits of
the padded batch prefill (`_prefill`, student_engine.py:679-737) and the logits of every eager decode step
(`_decode_step`, :795-832) when the engine feeds itself its own greedy tokens. `tests/test_plain.py` recomputes
all of it with the plain implementation and compares.
"""
import json
import sys
import tempfile
import types
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))

from tests import plain_qwen2 as plain  # noqa: E402
from tests.helpers import TINY_A, TINY_B, make_model_dir, random_tokens  # noqa: E402

CASES = [("tiny_a", TINY_A, 0, [5, 11, 17], 8), ("tiny_b", TINY_B, 1, [1, 7, 19, 33], 12)]


def main(reference_root: str) -> None:
    sys.path.insert(0, reference_root)
    import student_engine as se

    class StubTokenizer:
        pad_token_id = 0
        eos_token_id = 1
        pad_token = "<p>"
        eos_token = "<e>"
        padding_side = "right"

    se.AutoTokenizer = types.SimpleNamespace(from_pretrained=lambda *a, **k: StubTokenizer())
    out = {}
    for name, config, seed, lengths, n_decode in CASES:
        folder, _ = make_model_dir(config, seed, tempfile.mkdtemp(prefix="qf_golden_"))
        engine = se.StudentEngine(str(folder), device="cpu", dtype="float32", attn_implementation="eager",
                                  local_files_only=True)
        prompts = [random_tokens(config["vocab_size"], n, 1000 + n) for n in lengths]
        batch, longest = len(prompts), max(lengths)
        ids = torch.zeros(batch, longest, dtype=torch.long)
        mask = torch.zeros(batch, longest, dtype=torch.bool)
        for b, p in enumerate(prompts):
            ids[b, :len(p)] = torch.tensor(p)
            mask[b, :len(p)] = True
        lens = torch.tensor(lengths)
        capacity = longest + n_decode
        with torch.inference_mode():
            logits, caches = engine._prefill(ids, mask, lens, cache_capacity=capacity, has_padding=True)
            steps = [logits]
            cache_mask = torch.zeros(batch, capacity, dtype=torch.bool)
            cache_mask[:, :longest] = mask
            current = torch.argmax(logits, dim=-1)
            generated = [current.tolist()]
            for step in range(n_decode):
                slot = longest + step
                cache_mask[:, slot] = True
                logits = engine._decode_step(current, lens + step, caches, slot, cache_mask, True)
                steps.append(logits)
                current = torch.argmax(logits, dim=-1)
                generated.append(current.tolist())
        columns = list(range(0, config["vocab_size"], config["vocab_size"] // 24))[:24]
        out[name] = dict(seed=seed, prompts=prompts, n_decode=n_decode,
                         generated=[[generated[s][b] for s in range(n_decode + 1)] for b in range(batch)],
                         columns=columns,
                         logits=[[[round(float(steps[s][b][c]), 7) for c in columns] for s in range(n_decode + 1)]
                                 for b in range(batch)],
                         peak=[[round(float(steps[s][b].max()), 7) for s in range(n_decode + 1)]
                               for b in range(batch)])
    target = Path(__file__).with_name("reference_outputs.json")
    target.write_text(json.dumps(out, separators=(",", ":")))
    print(f"wrote {target} ({target.stat().st_size} bytes)")


if __name__ == "__main__":
    main(sys.argv[1])
