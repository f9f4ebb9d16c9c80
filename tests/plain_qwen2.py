"""Plain, slow implementation of the dense GQA Qwen2 decoder: the tests' oracle.

Whole sequences, no cache, one function for each part, no code shared with the
package under test. Every function restates a formula of the reference engine
and cites where it stands there (paths are relative to the reference project;
`SE` = student_engine.py, `LW` = utils/load_weights.py).

Numerics: the arithmetic runs in `dtype` (float64 by default, so that the oracle
is closer to the exact result than either engine precision). Two places follow
the reference's 32-bit choices on purpose because they change the *value*, not
just the rounding: the rotary frequency table and the rotation angle are formed
in float32 (SE:362-363, SE:548), and only then widened.

The reference has no sliding window (it ignores `use_sliding_window`,
`sliding_window`, `max_window_layers`: SE:327-349). The `window` argument below is
this library's own extension of the causal mask (SE:590-597) and says so there.
"""
from __future__ import annotations

from typing import Mapping, Sequence

import torch

Tensor = torch.Tensor


# --------------------------------------------------------------------------- config

def read_sizes(config: Mapping) -> dict:
    """Typed reads with the reference's defaults (SE:327-349).

    The reference computes head_dim = hidden // heads and ignores a `head_dim`
    key (SE:338); an explicit key is honoured here only if present, which agrees
    with it whenever the two are equal, as they are for every Qwen2.5 size.
    """
    hidden = int(config["hidden_size"])
    heads = int(config["num_attention_heads"])
    kv_heads = int(config.get("num_key_value_heads", heads))
    head_dim = int(config.get("head_dim") or hidden // heads)
    layers = int(config["num_hidden_layers"])
    use_window = bool(config.get("use_sliding_window", False))
    window = config.get("sliding_window")
    first_windowed = config.get("max_window_layers")
    first_windowed = layers if first_windowed is None else int(first_windowed)
    windows = [
        int(window) if (use_window and window is not None and i >= first_windowed) else 0
        for i in range(layers)
    ]
    return dict(
        hidden=hidden,
        inter=int(config["intermediate_size"]),
        layers=layers,
        heads=heads,
        kv_heads=kv_heads,
        head_dim=head_dim,
        eps=float(config.get("rms_norm_eps", 1e-6)),
        theta=float(config.get("rope_theta", 10000.0)),
        windows=windows,
    )


# --------------------------------------------------------------------------- parts

def rms_norm(x: Tensor, weight: Tensor, eps: float) -> Tensor:
    """x * rsqrt(mean(x^2) + eps) * w  (SE:530-535)."""
    variance = x.square().mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(variance + eps) * weight


def rope_inv_freq(head_dim: int, theta: float) -> Tensor:
    """inv_freq_j = 1 / theta^(2j/D), j = 0..D/2-1, formed in float32 (SE:362-363)."""
    idx = torch.arange(0, head_dim, 2, dtype=torch.float32)
    return 1.0 / (theta ** (idx / head_dim))


def rope_cos_sin(positions: Tensor, head_dim: int, theta: float, dtype) -> tuple[Tensor, Tensor]:
    """angle = float32(pos) * inv_freq in float32, duplicated over both halves (SE:548-551)."""
    angle = positions.to(torch.float32).unsqueeze(-1) * rope_inv_freq(head_dim, theta)
    emb = torch.cat((angle, angle), dim=-1).to(dtype)
    return emb.cos(), emb.sin()


def rotate_half(x: Tensor) -> Tensor:
    """[x1, x2] -> [-x2, x1] over the last axis (SE:537-540)."""
    first, second = x.chunk(2, dim=-1)
    return torch.cat((-second, first), dim=-1)


def apply_rope(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    """x * cos + rotate_half(x) * sin; x is [heads, S, D], cos/sin [S, D] (SE:552-553)."""
    return x * cos + rotate_half(x) * sin


def project_qkv(x: Tensor, w: Mapping[str, Tensor], prefix: str, heads: int, kv_heads: int, head_dim: int):
    """q/k/v = x W^T + b, each viewed as [heads, S, D] (SE:505-520, SE:563-575)."""
    seq = x.shape[0]
    q = x @ w[prefix + "q_proj.weight"].T + w[prefix + "q_proj.bias"]
    k = x @ w[prefix + "k_proj.weight"].T + w[prefix + "k_proj.bias"]
    v = x @ w[prefix + "v_proj.weight"].T + w[prefix + "v_proj.bias"]
    q = q.view(seq, heads, head_dim).transpose(0, 1)
    k = k.view(seq, kv_heads, head_dim).transpose(0, 1)
    v = v.view(seq, kv_heads, head_dim).transpose(0, 1)
    return q, k, v


def attention(q: Tensor, k: Tensor, v: Tensor, window: int = 0) -> Tensor:
    """Dense causal softmax attention with grouped heads (SE:579-599).

    q [NH,S,D], k/v [KVH,S,D]. Query head i reads kv head i // G (repeat_interleave,
    SE:587-588); scores scaled by D^-1/2 (SE:589); key j visible to query i iff
    j <= i (SE:590-596). `window` > 0 (this library's extension) also hides keys
    with j <= i - window.
    """
    heads, seq, head_dim = q.shape
    groups = heads // k.shape[0]
    k = k.repeat_interleave(groups, dim=0)
    v = v.repeat_interleave(groups, dim=0)
    scores = (q @ k.transpose(-2, -1)) * (head_dim ** -0.5)
    i = torch.arange(seq).unsqueeze(1)
    j = torch.arange(seq).unsqueeze(0)
    visible = j <= i
    if window > 0:
        visible = visible & (j > i - window)
    scores = scores.masked_fill(~visible, float("-inf"))
    return torch.softmax(scores, dim=-1) @ v


def swiglu_mlp(x: Tensor, w: Mapping[str, Tensor], prefix: str) -> Tensor:
    """(silu(x Wg^T) * (x Wu^T)) Wd^T, no biases (SE:523-527, SE:663-666)."""
    gate = x @ w[prefix + "gate_proj.weight"].T
    up = x @ w[prefix + "up_proj.weight"].T
    return (gate * torch.sigmoid(gate) * up) @ w[prefix + "down_proj.weight"].T


def decoder_layer(h: Tensor, w: Mapping[str, Tensor], index: int, sizes: dict, cos: Tensor, sin: Tensor) -> Tensor:
    """Pre-norm block: h += attn(norm1(h)); h += mlp(norm2(h))  (SE:696-731)."""
    p = f"model.layers.{index}."
    n = rms_norm(h, w[p + "input_layernorm.weight"], sizes["eps"])
    q, k, v = project_qkv(n, w, p + "self_attn.", sizes["heads"], sizes["kv_heads"], sizes["head_dim"])
    q = apply_rope(q, cos, sin)
    k = apply_rope(k, cos, sin)
    ctx = attention(q, k, v, sizes["windows"][index])
    ctx = ctx.transpose(0, 1).reshape(h.shape[0], sizes["heads"] * sizes["head_dim"])
    h = h + ctx @ w[p + "self_attn.o_proj.weight"].T
    n = rms_norm(h, w[p + "post_attention_layernorm.weight"], sizes["eps"])
    return h + swiglu_mlp(n, w, p + "mlp.")


# --------------------------------------------------------------------------- model

def forward_logits(config: Mapping, weights: Mapping[str, Tensor], token_ids: Sequence[int],
                   dtype=torch.float64) -> Tensor:
    """Logits at every position of one whole sequence, [S, V].

    embed (SE:690) -> layers -> final norm (SE:733) -> head (SE:736); the head is
    `lm_head.weight` when the file has one, else the embedding table (SE:359).
    Positions are 0..S-1 (SE:691-692).
    """
    sizes = read_sizes(config)
    w = {name: t.to(dtype) for name, t in weights.items()}
    ids = torch.as_tensor(list(token_ids), dtype=torch.long)
    h = w["model.embed_tokens.weight"][ids]
    cos, sin = rope_cos_sin(torch.arange(len(ids)), sizes["head_dim"], sizes["theta"], dtype)
    for index in range(sizes["layers"]):
        h = decoder_layer(h, w, index, sizes, cos, sin)
    h = rms_norm(h, w["model.norm.weight"], sizes["eps"])
    head = w.get("lm_head.weight", w["model.embed_tokens.weight"])
    return h @ head.T


def greedy_generate(config: Mapping, weights: Mapping[str, Tensor], prompt: Sequence[int], max_new_tokens: int,
                    stop_token_ids: Sequence[int] = (), dtype=torch.float64) -> list[int]:
    """argmax of the last position, appended, repeated (SE:1320, SE:1147-1160).

    The whole sequence is recomputed for every token: no cache. Stops after a stop
    token has been emitted (this library's extension; the reference never stops).
    """
    ids = list(prompt)
    out: list[int] = []
    for _ in range(max_new_tokens):
        nxt = int(torch.argmax(forward_logits(config, weights, ids, dtype)[-1]))
        out.append(nxt)
        ids.append(nxt)
        if nxt in stop_token_ids:
            break
    return out


# --------------------------------------------------------------------------- sampling

def gumbel_noise_u32(seed: int, sequence_id: int, step: int, vocab: int) -> Tensor:
    """The library's counter-based uniform bits, restated with Python integers.

    One 32-bit word per (seed, sequence, step, token id) from a fixed integer
    mixing function. The reference draws no random numbers (greedy only,
    SE:1320), so this has no counterpart there; it is restated here so that the
    sampling kernel can be checked value by value.
    """
    mask = 0xFFFFFFFF

    def mix(x: int) -> int:
        x &= mask
        x ^= x >> 16
        x = (x * 0x7FEB352D) & mask
        x ^= x >> 15
        x = (x * 0x846CA68B) & mask
        x ^= x >> 16
        return x

    key = mix((seed & mask) ^ 0x9E3779B9)
    key = mix(key ^ ((seed >> 32) & mask))
    key = mix(key ^ (sequence_id & mask))
    key = mix(key ^ ((sequence_id >> 32) & mask) ^ 0x85EBCA6B)
    key = mix(key ^ (step & mask))
    return torch.tensor([mix(key ^ mix(i ^ 0x27D4EB2F)) for i in range(vocab)], dtype=torch.int64)


def sample_token(logits: Tensor, temperature: float, seed: int, sequence_id: int, step: int) -> tuple[int, Tensor]:
    """Greedy (temperature 0: argmax, lowest id on ties; SE:1320) or Gumbel-max sampling.

    Gumbel-max: argmax_i(logit_i / T + g_i), g_i = -log(-log(u_i)), u_i in (0,1)
    from `gumbel_noise_u32`; this draws token i with probability softmax(logits/T)_i.
    Returns the token and the perturbed scores (float64) so that a test can accept
    a kernel's choice when two scores lie within rounding of each other.
    """
    logits = logits.to(torch.float64)
    if temperature <= 0.0:
        return int(torch.argmax(logits)), logits
    bits = gumbel_noise_u32(seed, sequence_id, step, logits.shape[-1])
    u = ((bits >> 9).to(torch.float64) + 0.5) * (1.0 / 8388608.0)
    scores = logits / temperature - torch.log(-torch.log(u))
    return int(torch.argmax(scores)), scores


# --------------------------------------------------------------------------- random weights

def tensor_names_and_shapes(config: Mapping) -> list[tuple[str, tuple[int, ...], str]]:
    """Every tensor the reference reads, by its name in the file (SE:357-359, SE:498-528).

    Returns (name, shape, kind) with kind in {"matrix", "norm", "bias"}; `lm_head.weight`
    only when `tie_word_embeddings` is false.
    """
    s = read_sizes(config)
    hidden, inter, d = s["hidden"], s["inter"], s["head_dim"]
    vocab = int(config["vocab_size"])
    out = [("model.embed_tokens.weight", (vocab, hidden), "matrix")]
    for i in range(s["layers"]):
        p = f"model.layers.{i}."
        out += [
            (p + "input_layernorm.weight", (hidden,), "norm"),
            (p + "self_attn.q_proj.weight", (s["heads"] * d, hidden), "matrix"),
            (p + "self_attn.q_proj.bias", (s["heads"] * d,), "bias"),
            (p + "self_attn.k_proj.weight", (s["kv_heads"] * d, hidden), "matrix"),
            (p + "self_attn.k_proj.bias", (s["kv_heads"] * d,), "bias"),
            (p + "self_attn.v_proj.weight", (s["kv_heads"] * d, hidden), "matrix"),
            (p + "self_attn.v_proj.bias", (s["kv_heads"] * d,), "bias"),
            (p + "self_attn.o_proj.weight", (hidden, s["heads"] * d), "matrix"),
            (p + "post_attention_layernorm.weight", (hidden,), "norm"),
            (p + "mlp.gate_proj.weight", (inter, hidden), "matrix"),
            (p + "mlp.up_proj.weight", (inter, hidden), "matrix"),
            (p + "mlp.down_proj.weight", (hidden, inter), "matrix"),
        ]
    out.append(("model.norm.weight", (hidden,), "norm"))
    if not bool(config.get("tie_word_embeddings", False)):
        out.append(("lm_head.weight", (vocab, hidden), "matrix"))
    return out


def random_weights(config: Mapping, seed: int, dtype=torch.float32) -> dict[str, Tensor]:
    """Seeded test weights: matrices and biases N(0, 0.02), norm weights 1 + N(0, 0.1).

    The reference has no random initialiser for its engine; this is the tests' own,
    independent of the package's, drawn with one CPU generator in name order.
    """
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape, kind in tensor_names_and_shapes(config):
        noise = torch.randn(shape, generator=gen, dtype=torch.float32)
        out[name] = (1.0 + 0.1 * noise if kind == "norm" else 0.02 * noise).to(dtype)
    return out


def logit_tolerance(reference: Tensor, rel: float, abs_: float) -> float:
    """abs_ + rel * max|reference|: the bound used when comparing logits."""
    return abs_ + rel * float(reference.abs().max())

