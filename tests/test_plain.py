"""The plain implementation checked on its own: against the reference engine's recorded outputs
(tests/golden), and part by part against properties that do not depend on any implementation."""
import json
from pathlib import Path

import pytest
import torch

from tests import plain_qwen2 as plain
from tests.helpers import TINY_A, TINY_B, TINY_W, random_tokens

GOLDEN = Path(__file__).parent / "golden" / "reference_outputs.json"


@pytest.mark.parametrize("name,config", [("tiny_a", TINY_A), ("tiny_b", TINY_B)])
def test_against_the_reference_engine(name, config):
    """The reference's own engine (CPU, float32, eager attention) on the same random weights: last-position logits of
    its padded batch prefill and of every decode step agree with the plain implementation run on whole sequences."""
    record = json.loads(GOLDEN.read_text())[name]
    weights = plain.random_weights(config, record["seed"])
    columns = record["columns"]
    for prompt, generated, logits, peak in zip(record["prompts"], record["generated"], record["logits"], record["peak"]):
        sequence = list(prompt) + generated[:-1]
        ours = plain.forward_logits(config, weights, sequence)[len(prompt) - 1:]
        assert ours.shape[0] == len(logits)
        theirs = torch.tensor(logits, dtype=torch.float64)
        assert float((ours[:, columns] - theirs).abs().max()) < 5e-6      # float32 engine against float64 oracle
        assert float((ours.max(-1).values - torch.tensor(peak, dtype=torch.float64)).abs().max()) < 5e-6
        assert ours.argmax(-1).tolist() == generated
        assert plain.greedy_generate(config, weights, prompt, len(generated)) == generated


def test_rms_norm():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    out = plain.rms_norm(x, torch.tensor([1.0, 2.0], dtype=torch.float64), 0.0)
    assert torch.allclose(out, torch.tensor([[3.0, 8.0]], dtype=torch.float64) / (12.5 ** 0.5))


def test_rope_is_a_rotation_by_relative_position():
    d, theta = 16, 10000.0
    assert float(plain.rope_inv_freq(4, theta)[1]) == pytest.approx(0.01, rel=1e-6)
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, 1, d, generator=g, dtype=torch.float64)
    k = torch.randn(1, 1, d, generator=g, dtype=torch.float64)

    def score(pq, pk):
        cq, sq = plain.rope_cos_sin(torch.tensor([pq]), d, theta, torch.float64)
        ck, sk = plain.rope_cos_sin(torch.tensor([pk]), d, theta, torch.float64)
        return float((plain.apply_rope(q, cq, sq) * plain.apply_rope(k, ck, sk)).sum())

    # depends on the distance only (to the float32 rounding of the angles, which the reference forms in float32)
    assert score(7, 3) == pytest.approx(score(14, 10), abs=1e-6)
    assert score(0, 0) == pytest.approx(float((q * k).sum()), abs=1e-12)  # position 0 is the identity
    c, s = plain.rope_cos_sin(torch.tensor([5]), d, theta, torch.float64)
    assert float(plain.apply_rope(q, c, s).norm()) == pytest.approx(float(q.norm()), abs=1e-12)
    # component j pairs with j + d/2 (split-half), not with j + 1
    e0 = torch.zeros(1, 1, d, dtype=torch.float64)
    e0[..., 0] = 1.0
    rotated = plain.apply_rope(e0, c, s)[0, 0]
    assert set(torch.nonzero(rotated.abs() > 1e-12).flatten().tolist()) == {0, d // 2}


def test_attention_is_causal_grouped_and_windowed():
    g = torch.Generator().manual_seed(1)
    q = torch.randn(4, 9, 8, generator=g, dtype=torch.float64)
    k = torch.randn(2, 9, 8, generator=g, dtype=torch.float64)
    v = torch.randn(2, 9, 8, generator=g, dtype=torch.float64)
    out = plain.attention(q, k, v)
    k2, v2 = k.clone(), v.clone()
    k2[:, 6:] += 1.0
    v2[:, 6:] -= 2.0
    assert torch.equal(plain.attention(q, k2, v2)[:, :6], out[:, :6])  # later keys never reach earlier queries
    assert torch.allclose(out[:, 0], v.repeat_interleave(2, dim=0)[:, 0])  # the first query sees only itself
    # heads 0,1 read kv head 0; heads 2,3 read kv head 1
    k3 = k.clone()
    k3[1] += 5.0
    changed = plain.attention(q, k3, v)
    assert torch.equal(changed[:2], out[:2]) and not torch.equal(changed[2:], out[2:])
    # a window of 3: the query at 8 sees keys 6, 7, 8 only
    win = plain.attention(q, k, v, window=3)
    k4, v4 = k.clone(), v.clone()
    k4[:, :6] += 3.0
    v4[:, :6] -= 3.0
    assert torch.allclose(plain.attention(q, k4, v4, window=3)[:, 8], win[:, 8])
    assert torch.allclose(plain.attention(q, k, v, window=100), out)


def test_swiglu_and_tensor_list():
    w = {"p.gate_proj.weight": torch.tensor([[1.0]], dtype=torch.float64),
         "p.up_proj.weight": torch.tensor([[2.0]], dtype=torch.float64),
         "p.down_proj.weight": torch.tensor([[3.0]], dtype=torch.float64)}
    x = torch.tensor([[0.5]], dtype=torch.float64)
    silu = 0.5 / (1 + torch.exp(torch.tensor(-0.5, dtype=torch.float64)))
    assert float(plain.swiglu_mlp(x, w, "p.")) == pytest.approx(float(silu) * 1.0 * 3.0)
    assert len(plain.tensor_names_and_shapes(TINY_A)) == 2 * 12 + 2          # tied: no lm_head
    assert len(plain.tensor_names_and_shapes(TINY_B)) == 3 * 12 + 3
    assert plain.read_sizes(TINY_W)["windows"] == [0, 37, 37]


def test_sampling_reference():
    logits = torch.tensor([0.1, 2.0, 2.0, -1.0])
    assert plain.sample_token(logits, 0.0, 0, 0, 0)[0] == 1                  # ties: the lowest id
    bits = plain.gumbel_noise_u32(1, 2, 3, 1000)
    assert int(bits.min()) >= 0 and int(bits.max()) < 2 ** 32 and len(set(bits.tolist())) > 990
    assert not torch.equal(bits, plain.gumbel_noise_u32(1, 2, 4, 1000))
    counts = torch.zeros(4)
    for step in range(3000):
        counts[plain.sample_token(logits, 1.0, 9, 0, step)[0]] += 1
    assert float((counts / 3000 - torch.softmax(logits.double(), -1)).abs().max()) < 0.03
