"""Decode steps of a few rows at layer widths beyond the presets': one decoder layer and the head at the widths of the
larger published Qwen2.5 models (5120 / 13824 with 40 query and 8 key-value heads of 128; 8192 / 29568 with 64 and 8),
and at a width that is no multiple of 32 with more weight tiles than one wave of blocks holds (1000 / 8000). At each,
steps of 16, 9, 8 and 1 rows run launch by launch and from a captured decode graph, and every step's logits are
compared with the plain implementation. Whatever the fused weight-streaming kernels do not take must run on the
unfused kernels: no step may raise."""
import json

import pytest
import torch

from tests import plain_qwen2 as plain
from tests.helpers import random_tokens

pytestmark = pytest.mark.gpu

WIDE = {
    "w5120": dict(hidden_size=5120, intermediate_size=13824, num_attention_heads=40, num_key_value_heads=8, head_dim=128),
    "w8192": dict(hidden_size=8192, intermediate_size=29568, num_attention_heads=64, num_key_value_heads=8, head_dim=128),
    "w4096": dict(hidden_size=4096, intermediate_size=11008, num_attention_heads=32, num_key_value_heads=32, head_dim=128),
    "w1000": dict(hidden_size=1000, intermediate_size=8000, num_attention_heads=10, num_key_value_heads=2, head_dim=64),
    # at 9 rows and more this one's gate/up product (90 MB) runs on the unfused kernels while its down product stays fused
    "w2048": dict(hidden_size=2048, intermediate_size=11008, num_attention_heads=16, num_key_value_heads=2, head_dim=128),
}
CHECKED = (0, 7, 8, 15)   # the sequences whose logits are compared (row 0 is in every step, row 15 only in the widest)
ROW_COUNTS = (16, 9, 8, 1)


def bound_of(ref: torch.Tensor) -> float:
    return 2e-2 + 4e-2 * float(ref.abs().max())


@pytest.mark.parametrize("name", list(WIDE))
def test_decode_steps_at_wide_layers(name, tmp_path):
    from qwenforge_b200.engine import Model
    from qwenforge_b200.engine.graphs import DecodeGraph
    from qwenforge_b200.sampling import Sampler
    from qwenforge_b200.weights import save_safetensors
    config = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=512, num_hidden_layers=1,
                  rms_norm_eps=1e-6, rope_theta=1000000.0, max_position_embeddings=256, tie_word_embeddings=True,
                  hidden_act="silu", use_sliding_window=False, torch_dtype="bfloat16", **WIDE[name])
    # weights that bfloat16 holds exactly, so that the comparison sees the arithmetic and not the storage rounding
    weights = {k: v.bfloat16().float() for k, v in plain.random_weights(config, 21).items()}
    (tmp_path / "config.json").write_text(json.dumps(config))
    save_safetensors(tmp_path / "model.safetensors", {k: v.bfloat16() for k, v in weights.items()})
    model = Model.from_dir(tmp_path, torch.bfloat16, "cuda")
    cache = model.new_cache(64 * 16, 16)
    seqs = [random_tokens(512, 3 + (5 * i) % 23, 800 + i) for i in range(16)]
    slots = [cache.open() for _ in seqs]
    cache.reserve([(slot, 64) for slot in slots])
    model.step(cache, list(zip(slots, seqs)))
    fed = [random_tokens(512, 2 * len(ROW_COUNTS), 900 + i) for i in range(16)]   # the tokens the decode steps feed
    got = {i: [] for i in CHECKED}
    # launch by launch
    for step, rows in enumerate(ROW_COUNTS):
        logits = model.step(cache, [(slots[i], [fed[i][step]]) for i in range(rows)])
        model.raise_on_kernel_error()
        for i in CHECKED:
            if i < rows:
                seqs[i].append(fed[i][step])
                got[i].append((len(seqs[i]) - 1, logits[i].float().cpu()))
        for i in range(rows):
            if i not in CHECKED:
                seqs[i].append(fed[i][step])
    # from a captured graph: the graph feeds back its own greedy tokens, so each replay's input is read from it
    sampler = Sampler()
    for step, rows in enumerate(ROW_COUNTS):
        cache.flush()
        graph = DecodeGraph(model, cache, rows, 64, sampler)
        graph.capture()
        tokens = [fed[i][len(ROW_COUNTS) + step] for i in range(rows)]
        graph.load(slots[:rows], tokens, [len(seqs[i]) for i in range(rows)], [1] * rows, [1 << 30] * rows,
                   list(range(rows)), [])
        for replay in range(2):
            produced = graph.run(1)[0]
            model.raise_on_kernel_error()
            for i in range(rows):
                seqs[i].append(tokens[i])
                cache.advance(slots[i], 1)
                if i in CHECKED:
                    got[i].append((len(seqs[i]) - 1, graph.last_logits[i].float().cpu()))
            tokens = produced[:rows]
        del graph
    for i in CHECKED:
        ref = plain.forward_logits(config, weights, seqs[i], dtype=torch.float32)
        for position, logits in got[i]:
            err = float((logits.double() - ref[position].double()).abs().max())
            assert err <= bound_of(ref), f"{name} sequence {i} position {position}: {err:.3e} > {bound_of(ref):.3e}"
    for slot in slots:
        cache.close(slot)


def test_the_planner_answers_for_what_the_launch_does():
    """`skinny_gemm_takes` is the library's own planning: for a grid of shapes, a yes launches and a no raises."""
    from qwenforge_b200 import ops
    torch.manual_seed(0)
    for k, n, m in [(5120, 7168, 16), (5120, 7168, 8), (8192, 10240, 1), (8192, 10240, 16), (1000, 16000, 4),
                    (1000, 1152, 4), (896, 1152, 16), (3584, 4608, 16), (4096, 12288, 9), (29568, 8192, 16)]:
        w = (torch.randn(n, k, device="cuda") * 0.02).bfloat16()
        hidden = torch.randn(m, k, device="cuda")
        norm_w = torch.ones(k, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        for norm in (True, False):
            takes = ops.skinny_gemm_takes(m, w, ops.EPI_PLAIN, norm)
            kwargs = dict(hidden=hidden, norm_weight=norm_w, eps=1e-6) if norm else dict(x=hidden.bfloat16())
            if takes:
                ops.skinny_gemm(ops.EPI_PLAIN, w, out=out, **kwargs)
                x = hidden.double()
                x = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-6) if norm else hidden.bfloat16().double()
                ref = x @ w.double().t()
                assert float((out.double() - ref).abs().max()) <= 2e-2 + 2e-2 * float(ref.abs().max()), (k, n, m, norm)
            else:
                with pytest.raises(ops.KernelError):
                    ops.skinny_gemm(ops.EPI_PLAIN, w, out=out, **kwargs)
    torch.cuda.synchronize()
