"""Plain PyTorch references of every CUDA kernel, with the kernels' own signatures.

Each function states in tensor operations what its kernel computes; the `-m gpu` tests compare the
two on the same inputs. The functions work on any device, so the CPU tests can also put them in
the kernels' place (`conftest.reference_kernels`) to exercise the step function, the cache and the
generation loop without a GPU. They are test code: the package never imports them.
"""
from __future__ import annotations

import torch

from tests import plain_qwen2 as plain

PAGE = 64


def _f(t):
    return t.to(torch.float64)


def embed_gather(ids, table, out, err):
    out.copy_(table[ids.long()].to(torch.float32))


def gather_rows(hidden, delta, rows, out, err):
    picked = hidden[rows.long()]
    if delta is not None:
        picked = picked + delta[rows.long()].to(torch.float32)
    out.copy_(picked)


def gather_rows_norm(hidden, delta, rows, weight, eps, out, err):
    picked = hidden[rows.long()]
    if delta is not None:
        picked = picked + delta[rows.long()].to(torch.float32)
    x = _f(picked)
    out.copy_((x * torch.rsqrt(x.square().mean(-1, keepdim=True) + eps) * _f(weight)).to(out.dtype))


def add_rms_norm(hidden, delta, weight, eps, out):
    if delta is not None:
        hidden += delta.to(torch.float32)
    x = _f(hidden)
    normed = x * torch.rsqrt(x.square().mean(-1, keepdim=True) + eps) * _f(weight)
    out.copy_(normed.to(out.dtype))


def gemm_f32(x, weight, bias, out):
    y = _f(x) @ _f(weight).T
    if bias is not None:
        y = y + _f(bias)
    out.copy_(y.to(out.dtype))


def linear(x, weight, bias=None, out=None, out_dtype=None):
    y = _f(x) @ _f(weight).T
    if bias is not None:
        y = y + _f(bias)
    y = y.to(out_dtype or x.dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y


def _kv_rows(site, slot, positions, head, which):
    """storage rows of `positions` (list) for one head: returns (page ids, offsets)."""
    pages = site.table[slot, torch.as_tensor(positions, device=site.table.device) // PAGE].long()
    offs = torch.as_tensor(positions, device=site.table.device) % PAGE
    return pages, offs


def rope_cache_write(qkv, tok_seq, tok_pos, slots, inv_freq, rot_dim, n_heads, q_out, site, write_cache, err, bias=None):
    n = qkv.shape[0]
    d, kvh = site.head_dim, site.kv_heads
    x = _f(qkv)
    if bias is not None:
        x = x + _f(bias)
    q = x[:, :n_heads * d].reshape(n, n_heads, d).clone()
    k = x[:, n_heads * d:(n_heads + kvh) * d].reshape(n, kvh, d).clone()
    v = x[:, (n_heads + kvh) * d:].reshape(n, kvh, d)
    if inv_freq is not None and rot_dim > 0:
        angle = (tok_pos.to(torch.float32).unsqueeze(-1) * inv_freq.to(torch.float32)).to(torch.float64)
        cos, sin = angle.cos().unsqueeze(1), angle.sin().unsqueeze(1)
        half = rot_dim // 2
        for t in (q, k):
            x1, x2 = t[..., :half].clone(), t[..., half:rot_dim].clone()
            t[..., :half] = x1 * cos - x2 * sin
            t[..., half:rot_dim] = x2 * cos + x1 * sin
    q_out.copy_(q.reshape(n, n_heads * d).to(q_out.dtype))
    if not write_cache:
        return
    for t in range(n):
        slot = int(slots[int(tok_seq[t])])
        if slot < 0:
            continue
        pos = int(tok_pos[t])
        page = int(site.table[slot, pos // PAGE])
        assert page >= 0, "reference: write to a page that is not held"
        site.storage[page, 0, :, pos % PAGE, :] = k[t].to(site.storage.dtype)
        site.storage[page, 1, :, pos % PAGE, :] = v[t].to(site.storage.dtype)


def gather_kv(site, slot, lo, hi):
    """Keys and values of positions lo..hi-1 of `slot`: two [kv_heads, hi-lo, head_dim] float64 tensors."""
    pos = torch.arange(lo, hi, device=site.table.device)
    pages = site.table[slot, pos // PAGE].long()
    assert bool((pages >= 0).all()), "reference: read of a page that is not held"
    k = site.storage[pages, 0, :, pos % PAGE, :]  # [n, kvh, d]
    v = site.storage[pages, 1, :, pos % PAGE, :]
    return _f(k).transpose(0, 1), _f(v).transpose(0, 1)


def attention_generic(q, out, cu_q, tok_pos, slots, site, n_heads, n_seqs, max_q_len, scale, window, err, scratch=None, max_kv_len=None):
    d, kvh = site.head_dim, site.kv_heads
    groups = n_heads // kvh
    for s in range(n_seqs):
        b, e = int(cu_q[s]), int(cu_q[s + 1])
        slot = int(slots[s])
        if slot < 0:
            out[b:e] = 0
            continue
        for t in range(b, e):
            p = int(tok_pos[t])
            lo = max(0, p - window + 1) if window > 0 else 0
            k, v = gather_kv(site, slot, lo, p + 1)
            qt = _f(q[t]).view(n_heads, d)
            k = k.repeat_interleave(groups, dim=0)
            v = v.repeat_interleave(groups, dim=0)
            scores = torch.einsum("hd,hjd->hj", qt, k) * scale
            ctx = torch.einsum("hj,hjd->hd", torch.softmax(scores, -1), v)
            out[t] = ctx.reshape(-1).to(out.dtype)


def swiglu(gate_up, out):
    inter = gate_up.shape[1] // 2
    g, u = _f(gate_up[:, :inter]), _f(gate_up[:, inter:])
    out.copy_((g * torch.sigmoid(g) * u).to(out.dtype))


def sample(logits, temperature, seed, seq_ids, steps, out, scratch=None):
    for r in range(logits.shape[0]):
        token, _ = plain.sample_token(logits[r].cpu(), temperature, seed,
                                      int(seq_ids[r]) if seq_ids is not None else 0,
                                      int(steps[r]) if steps is not None else 0)
        out[r] = token


ALL = dict(embed_gather=embed_gather, gather_rows=gather_rows, gather_rows_norm=gather_rows_norm, add_rms_norm=add_rms_norm, gemm_f32=gemm_f32,
           linear=linear, rope_cache_write=rope_cache_write, attention_generic=attention_generic, swiglu=swiglu,
           sample=sample)
