"""Shared helpers of the tests: tiny configurations, model folders in temporary places, tolerances."""
from __future__ import annotations

import tempfile
from pathlib import Path

import torch

from tests import plain_qwen2 as plain

# Two tiny configurations that differ in every size and option, and a third with a sliding window.
TINY_A = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=256, hidden_size=64, intermediate_size=128,
    num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6,
    rope_theta=10000.0, max_position_embeddings=384, tie_word_embeddings=True, hidden_act="silu",
    use_sliding_window=False, torch_dtype="float32")
TINY_B = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=384, hidden_size=120, intermediate_size=200,
    num_hidden_layers=3, num_attention_heads=5, num_key_value_heads=1, head_dim=24, rms_norm_eps=1e-5,
    rope_theta=1000000.0, max_position_embeddings=512, tie_word_embeddings=False, hidden_act="silu",
    use_sliding_window=False, torch_dtype="float32")
# windowed: layers 1.. see the last 37 positions only (not a multiple of the page or tile sizes)
TINY_W = dict(TINY_B, num_hidden_layers=3, use_sliding_window=True, sliding_window=37, max_window_layers=1,
              num_attention_heads=6, num_key_value_heads=3, hidden_size=96, head_dim=16, intermediate_size=88,
              vocab_size=320, rms_norm_eps=3e-6, rope_theta=50000.0)
# a mid-sized configuration with the head size of the real models, for the tensor-core kernels
SMALL_64 = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=1000, hidden_size=448, intermediate_size=616,
    num_hidden_layers=2, num_attention_heads=7, num_key_value_heads=1, head_dim=64, rms_norm_eps=1e-6,
    rope_theta=1000000.0, max_position_embeddings=2048, tie_word_embeddings=True, hidden_act="silu",
    use_sliding_window=False, torch_dtype="float32")
SMALL_128 = dict(SMALL_64, hidden_size=512, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                 intermediate_size=760, vocab_size=777, tie_word_embeddings=False, num_hidden_layers=2)

CONFIGS = {"tiny_a": TINY_A, "tiny_b": TINY_B, "tiny_w": TINY_W}


def make_model_dir(config: dict, seed: int, folder=None, store_dtype=torch.float32) -> tuple[Path, dict]:
    """Write config.json + model.safetensors with the TESTS' own random weights (not the package's
    random mode). Returns the folder and the float32 weights."""
    import json

    from qwenforge_b200.weights import save_safetensors

    folder = Path(folder or tempfile.mkdtemp(prefix="qf_model_"))
    folder.mkdir(parents=True, exist_ok=True)
    weights = plain.random_weights(config, seed)
    (folder / "config.json").write_text(json.dumps(config))
    save_safetensors(folder / "model.safetensors", {k: v.to(store_dtype) for k, v in weights.items()})
    return folder, weights


def random_tokens(vocab: int, length: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (length,), generator=g).tolist()


def max_err(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.double().cpu() - b.double().cpu()).abs().max())


# Tolerances. float32: the engine rounds every activation to float32 between kernels and sums in float32;
# the oracle is float64. bfloat16: weights and activations carry 8 bits of mantissa.
F32_REL, F32_ABS = 2e-5, 2e-6
BF16_REL, BF16_ABS = 4e-2, 2e-2


def assert_logits_close(got: torch.Tensor, ref: torch.Tensor, dtype: torch.dtype, what: str = "") -> None:
    rel, abs_ = (F32_REL, F32_ABS) if dtype == torch.float32 else (BF16_REL, BF16_ABS)
    bound = plain.logit_tolerance(ref, rel, abs_)
    err = max_err(got, ref)
    assert err <= bound, f"{what}: max |diff| {err:.3e} exceeds {bound:.3e}"
