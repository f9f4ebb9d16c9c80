"""Each CUDA kernel alone against its plain reference (tests/kernel_refs.py), at sizes other than the
engine's: odd widths, head sizes 16/24/40/64/128, group sizes 1/5/7/33, lengths around page and tile edges."""
import math

import pytest
import torch

from tests import kernel_refs as ref
from tests.helpers import max_err

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, scale=1.0):
    return (2e-5 if dtype == torch.float32 else 2e-2) * scale


@pytest.fixture(scope="module")
def ops():
    from qwenforge_b200 import ops
    return ops


def err_word():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vocab,width,n", [(37, 50, 9), (1000, 896, 33), (5, 7, 1)])
def test_embed_gather(ops, dtype, vocab, width, n):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(vocab, width, generator=g).to(dtype).to(DEV)
    ids = torch.randint(0, vocab, (n,), generator=g, dtype=torch.int32).to(DEV)
    out = torch.empty(n, width, device=DEV)
    e = err_word()
    ops.embed_gather(ids, table, out, e)
    want = torch.empty_like(out)
    ref.embed_gather(ids, table, want, None)
    assert torch.equal(out, want) and int(e) == 0
    ids[0] = vocab  # out of range: flagged, never read
    ops.embed_gather(ids, table, out, e)
    assert int(e) & ops.ERR_TOKEN_RANGE


@pytest.mark.parametrize("dtype", DTYPES)
def test_gather_rows(ops, dtype):
    g = torch.Generator().manual_seed(1)
    hidden = torch.randn(19, 70, generator=g).to(DEV)
    delta = torch.randn(19, 70, generator=g).to(dtype).to(DEV)
    rows = torch.tensor([18, 0, 7, 7], dtype=torch.int32, device=DEV)
    out = torch.empty(4, 70, device=DEV)
    e = err_word()
    ops.gather_rows(hidden, delta, rows, out, e)
    assert torch.equal(out, hidden[rows.long()] + delta[rows.long()].float()) and int(e) == 0
    ops.gather_rows(hidden, None, rows, out, e)
    assert torch.equal(out, hidden[rows.long()])
    rows[1] = 19
    ops.gather_rows(hidden, None, rows, out, e)
    assert int(e) & ops.ERR_ROW_RANGE


@pytest.mark.parametrize("embed", [False, True])
def test_decode_advance(ops, embed):
    """The kernel that ends a decode step, alone and with the next step's embedding, against the rules written out:
    a live row records its token, feeds it back, moves on one position and one step, and retires on a stop token or a
    spent budget; a retired row records -1 and keeps its state; a full chunk records nothing and moves nothing."""
    rows, width, vocab, chunk = 5, 24, 40, 3
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    token_ids, tok_pos, slots = i32([1, 2, 3, 4, 5]), i32([10, 20, 30, 40, 50]), i32([0, -1, 2, 3, 4])
    steps, budgets, stop_ids = i32([1, 1, 1, 1, 6]), i32([9, 9, 9, 2, 9]), i32([33, 7, -1, -1])
    out_tokens, cursor = torch.full((chunk, rows), -7, dtype=torch.int32, device=DEV), i32([0])
    g = torch.Generator().manual_seed(4)
    table = torch.randn(vocab, width, generator=g).to(torch.bfloat16).to(DEV)
    hidden, ticket, e = torch.zeros(rows, width, device=DEV), i32([0]), err_word()
    def step(sampled):
        if embed:
            ops.decode_advance_embed(i32(sampled), token_ids, tok_pos, slots, steps, budgets, stop_ids, 4, out_tokens, cursor,
                                     table, hidden, ticket, e)
        else:
            ops.decode_advance(i32(sampled), token_ids, tok_pos, slots, steps, budgets, stop_ids, 4, out_tokens, cursor)
    step([11, 12, 7, 14, 15])      # row 2 draws a stop token, row 3 spends its budget, row 1 is a padding entry
    assert out_tokens[0].tolist() == [11, -1, 7, 14, 15] and int(cursor) == 1
    assert token_ids.tolist() == [11, 2, 7, 14, 15] and tok_pos.tolist() == [11, 20, 31, 41, 51]
    assert slots.tolist() == [0, -1, -1, -1, 4] and steps.tolist() == [2, 1, 2, 2, 7]
    step([21, 22, 23, 24, 33])     # the retired rows stay as they are; row 4 draws the other stop token
    assert out_tokens[1].tolist() == [21, -1, -1, -1, 33] and int(cursor) == 2
    assert token_ids.tolist() == [21, 2, 7, 14, 33] and slots.tolist() == [0, -1, -1, -1, -1]
    step([31, 0, 0, 0, 0])
    assert out_tokens[2].tolist() == [31, -1, -1, -1, -1] and int(cursor) == 3 and tok_pos[0].item() == 13
    step([39, 0, 0, 0, 0])         # the chunk is full: nothing is recorded, nothing moves
    assert int(cursor) == 3 and token_ids[0].item() == 31 and tok_pos[0].item() == 13 and steps[0].item() == 4
    if embed:
        assert int(ticket) == 0 and int(e) == 0
        assert torch.equal(hidden, table[token_ids.long()].float())
        token_ids[1] = vocab       # a token outside the table: zeros and the error word, as the embedding kernel does
        cursor.zero_()
        step([1, 1, 1, 1, 1])
        assert int(e) & ops.ERR_TOKEN_RANGE and float(hidden[1].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,eps", [(70, 1e-6), (896, 1e-5), (3584, 1e-6), (1, 1e-3), (5001, 1e-6)])
def test_gather_rows_norm(ops, dtype, width, eps):
    g = torch.Generator().manual_seed(3)
    hidden = (torch.randn(19, width, generator=g) * 3).to(DEV)
    delta = torch.randn(19, width, generator=g).to(dtype).to(DEV)
    weight = (1 + 0.1 * torch.randn(width, generator=g)).to(dtype).to(DEV)
    rows = torch.tensor([18, 0, 7, 7], dtype=torch.int32, device=DEV)
    e = err_word()
    for d in (delta, None):
        out = torch.empty(4, width, dtype=dtype, device=DEV)
        want = torch.empty(4, width, dtype=torch.float32, device=DEV)
        ops.gather_rows_norm(hidden, d, rows, weight, eps, out, e)
        ref.gather_rows_norm(hidden, d, rows, weight, eps, want, None)
        assert int(e) == 0
        assert max_err(out, want) <= (2e-2 if dtype == torch.bfloat16 else 2e-5) * max(1.0, float(want.abs().max()))
        assert torch.equal(out[2], out[3])
    rows[1] = 19
    ops.gather_rows_norm(hidden, None, rows, weight, eps, out, e)
    assert int(e) & ops.ERR_ROW_RANGE and float(out[1].float().abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,width,eps", [(5, 64, 1e-6), (3, 120, 1e-5), (17, 896, 1e-6), (2, 3584, 1e-6), (1, 1, 1e-3)])
def test_add_rms_norm(ops, dtype, rows, width, eps):
    g = torch.Generator().manual_seed(2)
    hidden = (torch.randn(rows, width, generator=g) * 3).to(DEV)
    delta = torch.randn(rows, width, generator=g).to(dtype).to(DEV)
    weight = (1 + 0.1 * torch.randn(width, generator=g)).to(dtype).to(DEV)
    for d in (delta, None):
        h1, h2 = hidden.clone(), hidden.clone()
        out = torch.empty(rows, width, dtype=dtype, device=DEV)
        want = torch.empty_like(out)
        ops.add_rms_norm(h1, d, weight, eps, out)
        ref.add_rms_norm(h2, d, weight, eps, want)
        assert torch.equal(h1, h2)  # the residual sum is a plain float32 addition
        assert max_err(out, want) <= tol(dtype) * float(want.float().abs().max())


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (7, 200, 120), (70, 65, 33), (33, 1152, 896), (130, 50, 4864), (16, 301, 1000), (17, 301, 1000)])
def test_gemm_f32(ops, m, n, k):
    g = torch.Generator().manual_seed(3)
    x = torch.randn(m, k, generator=g).to(DEV)
    w = (torch.randn(n, k, generator=g) * 0.05).to(DEV)
    b = torch.randn(n, generator=g).to(DEV)
    out = torch.empty(m, n, device=DEV)
    want = torch.empty_like(out)
    ops.gemm_f32(x, w, b, out)
    ref.gemm_f32(x, w, b, want)
    assert max_err(out, want) <= 1e-6 * math.sqrt(k) * float(want.abs().max()) + 1e-6
    # a row's result does not depend on the rows around it: bitwise
    one = torch.empty(1, n, device=DEV)
    ops.gemm_f32(x[m // 2:m // 2 + 1], w, b, one)
    assert torch.equal(one[0], out[m // 2])
    # strided input rows
    wide = torch.randn(m, k + 5, generator=g).to(DEV)
    ops.gemm_f32(wide[:, :k], w, None, out)
    ref.gemm_f32(wide[:, :k], w, None, want)
    assert max_err(out, want) <= 1e-6 * math.sqrt(k) * float(want.abs().max()) + 1e-6


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,inter", [(3, 200), (17, 4864), (1, 1)])
def test_swiglu(ops, dtype, rows, inter):
    g = torch.Generator().manual_seed(4)
    gu = (torch.randn(rows, 2 * inter, generator=g) * 2).to(dtype).to(DEV)
    out = torch.empty(rows, inter, dtype=dtype, device=DEV)
    want = torch.empty_like(out)
    ops.swiglu(gu, out)
    ref.swiglu(gu, want)
    assert max_err(out, want) <= tol(dtype) * max(1.0, float(want.float().abs().max()))


class FakeSite:
    """A paged key/value store like the cache's, with pages handed out in a scrambled order."""

    def __init__(self, n_slots, max_len, kvh, d, dtype, seed=0):
        per_seq = (max_len + 63) // 64
        n_pages = n_slots * per_seq + 3
        g = torch.Generator().manual_seed(seed)
        self.storage = torch.zeros(n_pages, 2, kvh, 64, d, dtype=dtype, device=DEV)
        perm = torch.randperm(n_pages, generator=g)[: n_slots * per_seq].to(torch.int32)
        self.table = perm.view(n_slots, per_seq).to(DEV)
        self.kv_heads, self.head_dim = kvh, d


def fill_site(site, slot, length, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    kvh, d = site.kv_heads, site.head_dim
    k = torch.randn(length, kvh, d, generator=g).to(dtype).to(DEV)
    v = torch.randn(length, kvh, d, generator=g).to(dtype).to(DEV)
    pos = torch.arange(length, device=DEV)
    pages = site.table[slot, pos // 64].long()
    site.storage[pages, 0, :, pos % 64, :] = k
    site.storage[pages, 1, :, pos % 64, :] = v


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,kvh,d,rot", [(4, 2, 16, 16), (5, 1, 24, 24), (7, 1, 64, 64), (4, 2, 128, 64), (3, 3, 40, 0)])
def test_rope_cache_write(ops, dtype, nh, kvh, d, rot):
    g = torch.Generator().manual_seed(5)
    q_lens, starts, slots = [3, 1, 70], [0, 63, 60], [2, -1, 0]
    site_a = FakeSite(3, 256, kvh, d, dtype)
    site_b = FakeSite(3, 256, kvh, d, dtype)
    site_b.table = site_a.table
    n = sum(q_lens)
    qkv = torch.randn(n, (nh + 2 * kvh) * d, generator=g).to(dtype).to(DEV)
    tok_seq = torch.tensor(sum(([i] * q for i, q in enumerate(q_lens)), []), dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor(sum((list(range(s, s + q)) for s, q in zip(starts, q_lens)), []), dtype=torch.int32, device=DEV)
    slots_t = torch.tensor(slots, dtype=torch.int32, device=DEV)
    inv_freq = None
    if rot:
        inv_freq = (1.0 / (10000.0 ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))).to(DEV)
    q1 = torch.empty(n, nh * d, dtype=dtype, device=DEV)
    q2 = torch.empty_like(q1)
    e = err_word()
    a = ops.KvSiteArgs(site_a.storage, site_a.table, kvh, d)
    ops.rope_cache_write(qkv, tok_seq, tok_pos, slots_t, inv_freq, rot, nh, q1, a, True, e)
    ref.rope_cache_write(qkv, tok_seq, tok_pos, slots_t, inv_freq, rot, nh, q2, site_b, True, None)
    assert int(e) == 0
    assert max_err(q1, q2) <= tol(dtype) * 5
    assert max_err(site_a.storage, site_b.storage) <= tol(dtype) * 5
    # without the write flag the cache stays as it is
    before = site_a.storage.clone()
    ops.rope_cache_write(qkv, tok_seq, tok_pos, slots_t, inv_freq, rot, nh, q1, a, False, e)
    assert torch.equal(before, site_a.storage)


def run_attention(ops, fn_name, dtype, nh, kvh, d, q_lens, starts, window, slots=None, seed=6, **more):
    n_seqs = len(q_lens)
    slots = slots if slots is not None else list(range(n_seqs))[::-1]
    max_len = max(s + q for s, q in zip(starts, q_lens))
    site = FakeSite(n_seqs, max_len, kvh, d, dtype, seed)
    for slot, s, q in zip(slots, starts, q_lens):
        if slot >= 0:
            fill_site(site, slot, s + q, seed + slot, dtype)
    g = torch.Generator().manual_seed(seed)
    n = sum(q_lens)
    q = torch.randn(n, nh * d, generator=g).to(dtype).to(DEV)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor(sum((list(range(s, s + ql)) for s, ql in zip(starts, q_lens)), []), dtype=torch.int32, device=DEV)
    slots_t = torch.tensor(slots, dtype=torch.int32, device=DEV)
    out = torch.full((n, nh * d), 7.0, dtype=dtype, device=DEV)
    want = torch.empty_like(out)
    e = err_word()
    args = ops.KvSiteArgs(site.storage, site.table, kvh, d)
    scale = d ** -0.5
    getattr(ops, fn_name)(q, out, cu, tok_pos, slots_t, args, nh, n_seqs, max(q_lens), scale, window, e, **more)
    ref.attention_generic(q, want, cu, tok_pos, slots_t, site, nh, n_seqs, max(q_lens), scale, window, None)
    assert int(e) == 0
    return out, want


ATTN_SHAPES = [
    # nh, kvh, d, q_lens, starts, window
    (4, 2, 16, [5, 11, 17], [0, 0, 0], 0),
    (5, 1, 24, [1, 7, 19, 33], [0, 0, 0, 0], 0),
    (5, 1, 24, [1, 1, 1], [0, 63, 200], 0),              # decode at page edges
    (14, 2, 64, [130, 3], [0, 125], 0),                  # a continuation that crosses a page
    (4, 4, 40, [70], [10], 0),                           # no grouping, odd head size
    (33, 1, 16, [9, 2], [5, 0], 0),                      # a group larger than a block's rows
    (6, 3, 16, [100, 1, 40], [0, 90, 30], 37),           # window, not a multiple of anything
    (8, 2, 128, [65, 1], [0, 300], 64),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,kvh,d,q_lens,starts,window", ATTN_SHAPES)
def test_attention_generic(ops, dtype, nh, kvh, d, q_lens, starts, window):
    out, want = run_attention(ops, "attention_generic", dtype, nh, kvh, d, q_lens, starts, window)
    assert max_err(out, want) <= tol(dtype) * 3


GENERIC_DECODE_SHAPES = [
    # nh, kvh, d, starts (one token per sequence), window, slots
    # (the longest sequence first: it is also run alone)
    (14, 2, 64, [1500, 0, 255, 256, 257, 700], 0, None),
    (5, 1, 24, [1023, 511, 512, 3], 0, None),
    (6, 3, 16, [900, 300, 40, 256], 290, None),          # a window that crosses chunks of keys
    (33, 1, 16, [600, 10], 0, None),                     # a group larger than a block's rows
    (4, 2, 40, [800, 5, 400], 0, [1, -1, 0]),            # a padding entry in the middle
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,kvh,d,starts,window,slots", GENERIC_DECODE_SHAPES)
def test_attention_generic_decode_in_chunks_of_keys(ops, dtype, nh, kvh, d, starts, window, slots):
    """One token per sequence over caches longer than one chunk of keys: a block per chunk and a fold, against the plain
    reference; and a row's result is bit for bit the same whatever else the batch holds (here: alone, with a far larger
    bound on the lengths, hence more chunks in the launch)."""
    n = len(starts)
    slots = slots if slots is not None else list(range(n))[::-1]
    site = FakeSite(n, max(starts) + 1, kvh, d, dtype, 6)
    for slot, s in zip(slots, starts):
        if slot >= 0:
            fill_site(site, slot, s + 1, 6 + slot, dtype)
    g = torch.Generator().manual_seed(6)
    q = torch.randn(n, nh * d, generator=g).to(dtype).to(DEV)
    cu = torch.arange(n + 1, dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor(starts, dtype=torch.int32, device=DEV)
    slots_t = torch.tensor(slots, dtype=torch.int32, device=DEV)
    out = torch.full((n, nh * d), 7.0, dtype=dtype, device=DEV)
    want = torch.empty_like(out)
    e = err_word()
    args = ops.KvSiteArgs(site.storage, site.table, kvh, d)
    scratch = ops.DecodeScratch(DEV)
    bound = max(starts) + 1
    ops.attention_generic(q, out, cu, tok_pos, slots_t, args, nh, n, 1, d ** -0.5, window, e, scratch=scratch, max_kv_len=bound)
    ref.attention_generic(q, want, cu, tok_pos, slots_t, site, nh, n, 1, d ** -0.5, window, None)
    assert int(e) == 0 and bound > ops.GENERIC_DECODE_CHUNK and scratch.part_o is not None     # the split form ran
    assert max_err(out, want) <= tol(dtype) * 3
    if -1 in slots:
        assert float(out[slots.index(-1)].abs().max()) == 0.0
    alone = torch.full((1, nh * d), 7.0, dtype=dtype, device=DEV)
    ops.attention_generic(q[:1].contiguous(), alone, cu[:2], tok_pos[:1], slots_t[:1], args, nh, 1, 1, d ** -0.5, window, e,
                          scratch=ops.DecodeScratch(DEV), max_kv_len=4 * bound)
    assert int(e) == 0 and torch.equal(alone[0], out[0])


def test_attention_generic_padding_entry(ops):
    out, want = run_attention(ops, "attention_generic", torch.float32, 4, 2, 16, [3, 2, 4], [0, 0, 7], 0, slots=[1, -1, 0])
    assert max_err(out, want) <= 1e-5
    assert float(out[3:5].abs().max()) == 0.0


def test_attention_generic_far_key_stands_out(ops):
    """One key far back among hundreds is made to dominate: the output must be that key's value."""
    dtype, nh, kvh, d, length = torch.float32, 2, 1, 32, 700
    site = FakeSite(1, length, kvh, d, dtype, 9)
    fill_site(site, 0, length, 3, dtype)
    far = 17
    page, off = int(site.table[0, far // 64]), far % 64
    site.storage[page, 0, 0, off] = 0
    site.storage[page, 0, 0, off, 0] = 50.0
    q = torch.zeros(1, nh * d, device=DEV)
    q[0, 0] = 40.0
    q[0, d] = 40.0
    out = torch.empty_like(q)
    cu = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    pos = torch.tensor([length - 1], dtype=torch.int32, device=DEV)
    slots = torch.tensor([0], dtype=torch.int32, device=DEV)
    e = err_word()
    ops.attention_generic(q, out, cu, pos, slots, ops.KvSiteArgs(site.storage, site.table, kvh, d), nh, 1, 1,
                          d ** -0.5, 0, e)
    value = site.storage[page, 1, 0, off]
    assert max_err(out[0, :d], value) < 1e-4 and max_err(out[0, d:], value) < 1e-4
    # with a window that excludes it, it must vanish
    ops.attention_generic(q, out, cu, pos, slots, ops.KvSiteArgs(site.storage, site.table, kvh, d), nh, 1, 1,
                          d ** -0.5, length - far - 1, e)
    assert max_err(out[0, :d], value) > 1e-2


@pytest.mark.parametrize("vocab", [5, 384, 151936])
def test_sample_greedy_and_gumbel(ops, vocab):
    from tests import plain_qwen2 as plain
    g = torch.Generator().manual_seed(8)
    rows = 6
    logits = (torch.randn(rows, vocab + 3, generator=g) * 3).to(DEV)[:, :vocab]  # strided rows
    logits[2, 1] = logits[2, vocab - 1] = 99.0  # a tie: the lowest id wins
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    ops.sample(logits, 0.0, 0, None, None, out)
    best = logits.argmax(-1).tolist()
    assert [t for r, t in enumerate(out.tolist()) if r != 2] == [t for r, t in enumerate(best) if r != 2]
    assert out[2].item() == 1
    seq_ids = torch.tensor([3, 1 << 40, 5, 3, 9, 0], dtype=torch.int64, device=DEV)
    steps = torch.tensor([0, 1, 2, 0, 7, 4], dtype=torch.int32, device=DEV)
    ops.sample(logits, 0.7, 1234, seq_ids, steps, out)
    n_check = rows if vocab < 100000 else 2
    for r in range(n_check):
        token, scores = plain.sample_token(logits[r].cpu(), 0.7, 1234, int(seq_ids[r]), int(steps[r]))
        # the kernel's logarithms are float32: accept its choice if its score is within rounding of the best
        assert float(scores[token] - scores[int(out[r])]) <= 1e-4, (r, token, int(out[r]))
    # the draw of a row depends on (seed, sequence, step) only: row 3 has the key of row 0 but other logits
    alone = torch.empty(1, dtype=torch.int32, device=DEV)
    ops.sample(logits[0:1], 0.7, 1234, seq_ids[0:1], steps[0:1], alone)
    assert alone.item() == out[0].item()


def test_sample_distribution(ops):
    """Over many steps the draws follow softmax(logits / T)."""
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0, 0.5]], device=DEV).repeat(4000, 1)
    seq_ids = torch.zeros(4000, dtype=torch.int64, device=DEV)
    steps = torch.arange(4000, dtype=torch.int32, device=DEV)
    out = torch.empty(4000, dtype=torch.int32, device=DEV)
    ops.sample(logits, 1.3, 77, seq_ids, steps, out)
    freq = torch.bincount(out.long().cpu(), minlength=5).double() / 4000
    want = torch.softmax(logits[0].double().cpu() / 1.3, -1)
    assert float((freq - want).abs().max()) < 0.03


# ------------------------------------------------------------------------------------------------ tensor-core attention

FAST_PREFILL_SHAPES = [
    # nh, kvh, d, q_lens, starts, window
    (14, 2, 64, [130, 3, 64], [0, 125, 0], 0),
    (7, 1, 64, [1, 65, 200], [0, 63, 1], 0),
    (4, 2, 128, [70, 129], [10, 0], 0),
    (6, 3, 32, [100, 1, 40], [0, 90, 30], 37),          # window
    (8, 2, 96, [65, 17], [300, 5], 64),
    (33, 1, 32, [9, 2], [5, 0], 0),
    (16, 2, 128, [257], [0], 100),
]


FAST_PREFILL_SHAPES += [
    (2, 1, 64, [1100], [0], 0),                        # 18 pages for the last tile: shared between the groups unevenly
    (2, 2, 128, [64, 700], [900, 0], 0),               # a short continuation over a long cache beside a long prompt
    (3, 1, 64, [600], [0], 200),                       # a window of a few pages
]


@pytest.mark.parametrize("max_kv_len", [64, None], ids=["one_group", "two_groups"])
@pytest.mark.parametrize("nh,kvh,d,q_lens,starts,window", FAST_PREFILL_SHAPES)
def test_attention_prefill(ops, nh, kvh, d, q_lens, starts, window, max_kv_len):
    """`max_kv_len` steers only how a tile's pages are shared among warps: a bound of one page keeps one group of warps
    per tile, no bound lets two groups take alternate pages and merge."""
    out, want = run_attention(ops, "attention_prefill", torch.bfloat16, nh, kvh, d, q_lens, starts, window, max_kv_len=max_kv_len)
    assert max_err(out, want) <= 3e-2


TC_PREFILL_SHAPES = [
    # nh, kvh, d, q_lens, starts, window
    (14, 2, 64, [130, 3, 64], [0, 125, 0], 0),
    (7, 1, 64, [1, 65, 200], [0, 63, 1], 0),
    (4, 2, 128, [70, 129], [10, 0], 0),
    (2, 1, 64, [700], [0], 0),                           # several blocks of rows, pages far left of the diagonal
    (3, 3, 64, [300, 128], [100, 64], 150),              # window across blocks of rows
    (16, 2, 128, [257], [0], 100),
    (2, 2, 128, [40], [1000], 0),                        # a short continuation over a long cache
]


TC_PREFILL_SHAPES += [
    (2, 1, 64, [1100], [0], 0),                          # 18 pages for the last tile: an odd share for the second block
    (2, 2, 128, [64, 700], [900, 0], 0),                 # a short continuation over a long cache beside a long prompt
    (3, 1, 64, [600, 1], [0, 0], 200),                   # a window of a few pages; a one-token sequence (one page, one block idle)
]


@pytest.mark.parametrize("max_kv_len", [64, None], ids=["one_block", "two_blocks"])
@pytest.mark.parametrize("nh,kvh,d,q_lens,starts,window", TC_PREFILL_SHAPES)
def test_attention_prefill_tc(ops, nh, kvh, d, q_lens, starts, window, max_kv_len):
    """One block per tile of 128 rows, or (few tiles of many pages: no bound given) two blocks of a cluster that take
    alternate pages and merge through distributed shared memory."""
    out, want = run_attention(ops, "attention_prefill_tc", torch.bfloat16, nh, kvh, d, q_lens, starts, window, max_kv_len=max_kv_len)
    assert max_err(out, want) <= 3e-2


def test_attention_prefill_tc_padding_entry_and_refusal(ops):
    out, want = run_attention(ops, "attention_prefill_tc", torch.bfloat16, 4, 2, 64, [3, 2, 70], [0, 0, 7], 0, slots=[1, -1, 0])
    assert max_err(out, want) <= 3e-2 and float(out[3:5].float().abs().max()) == 0.0
    with pytest.raises(ops.KernelError, match="head_dim 32"):
        run_attention(ops, "attention_prefill_tc", torch.bfloat16, 5, 1, 32, [4], [0], 0)


def test_attention_prefill_padding_entry_and_refusal(ops):
    out, want = run_attention(ops, "attention_prefill", torch.bfloat16, 4, 2, 64, [3, 2, 70], [0, 0, 7], 0, slots=[1, -1, 0])
    assert max_err(out, want) <= 3e-2 and float(out[3:5].float().abs().max()) == 0.0
    with pytest.raises(ops.KernelError, match="head_dim 24"):
        run_attention(ops, "attention_prefill", torch.bfloat16, 5, 1, 24, [4], [0], 0)


@pytest.mark.parametrize("fn_name", ["attention_prefill", "attention_prefill_tc"])
@pytest.mark.parametrize("d", [64, 128])
def test_attention_prefill_far_key_and_window_edge(ops, fn_name, d):
    """200 new rows continue a cache of 600 positions. One key is made to dominate every query's softmax, so each
    row's output must be that key's value: far left of the diagonal without a window; with a window of 150 the key at
    position 500 is the last one that row 649 sees and the first one that row 650 does not."""
    nh, kvh, start, q_len = 2, 1, 600, 200
    length = start + q_len
    for window, far in ((0, 37), (150, 500)):
        site = FakeSite(1, length, kvh, d, torch.bfloat16, 9)
        fill_site(site, 0, length, 3, torch.bfloat16)
        page, off = int(site.table[0, far // 64]), far % 64
        site.storage[page, 0, 0, off] = 0
        site.storage[page, 0, 0, off, 0] = 60.0
        q = torch.zeros(q_len, nh * d, dtype=torch.bfloat16, device=DEV)
        q[:, 0] = q[:, d] = 40.0
        out = torch.full_like(q, 7.0)
        cu = torch.tensor([0, q_len], dtype=torch.int32, device=DEV)
        pos = torch.arange(start, length, dtype=torch.int32, device=DEV)
        slots = torch.tensor([0], dtype=torch.int32, device=DEV)
        e = err_word()
        getattr(ops, fn_name)(q, out, cu, pos, slots, ops.KvSiteArgs(site.storage, site.table, kvh, d), nh, 1, q_len,
                              d ** -0.5, window, e)
        assert int(e) == 0
        value = site.storage[page, 1, 0, off].float()
        diff = (out.float().view(q_len, nh, d) - value).abs().amax(dim=(1, 2))   # per row
        sees = (pos.cpu() - far < window) if window else torch.ones(q_len, dtype=torch.bool)
        assert float(diff[sees.to(DEV)].max()) < 2e-2, f"{fn_name} d={d} window={window}: a row lost the dominant key"
        if window:
            assert int(sees.sum()) == 50 and float(diff[(~sees).to(DEV)].min()) > 0.1, \
                f"{fn_name} d={d}: a row beyond the window's edge still sees the key"


def run_decode(ops, nh, kvh, d, lengths, window, n_splits, slots=None, seed=12):
    n = len(lengths)
    slots = slots if slots is not None else list(range(n))[::-1]
    site = FakeSite(n, max(lengths), kvh, d, torch.bfloat16, seed)
    for slot, length in zip(slots, lengths):
        if slot >= 0:
            fill_site(site, slot, length, seed + slot, torch.bfloat16)
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(n, nh * d, generator=g).to(torch.bfloat16).to(DEV)
    cu = torch.arange(n + 1, dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor([length - 1 for length in lengths], dtype=torch.int32, device=DEV)
    slots_t = torch.tensor(slots, dtype=torch.int32, device=DEV)
    out = torch.full((n, nh * d), 7.0, dtype=torch.bfloat16, device=DEV)
    want = torch.empty_like(out)
    e = err_word()
    args = ops.KvSiteArgs(site.storage, site.table, kvh, d)
    scratch = ops.DecodeScratch(DEV)
    for _ in range(2):  # twice with the same scratch: the ticket counters must come back to zero
        out.fill_(7.0)
        ops.attention_decode(q, out, cu, tok_pos, slots_t, args, nh, n, d ** -0.5, window, n_splits, scratch, e)
    ref.attention_generic(q, want, cu, tok_pos, slots_t, site, nh, n, 1, d ** -0.5, window, None)
    assert int(e) == 0
    if n_splits > 1:
        assert int(scratch.counters.abs().max()) == 0
    return out, want


@pytest.mark.parametrize("n_splits", [1, 2, 5, 64])
@pytest.mark.parametrize("nh,kvh,d,lengths,window", [
    (14, 2, 64, [1, 64, 65, 700], 0),
    (7, 1, 64, [4096, 130], 0),
    (16, 4, 128, [300, 1, 129], 0),
    (40, 2, 32, [200, 77], 0),               # a group of 20: two chunks of query heads
    (6, 3, 96, [500, 36, 1], 37),            # window
    (8, 2, 128, [1000], 64),
])
def test_attention_decode(ops, nh, kvh, d, lengths, window, n_splits):
    out, want = run_decode(ops, nh, kvh, d, lengths, window, n_splits)
    assert max_err(out, want) <= 3e-2


@pytest.mark.parametrize("nh,kvh,d,n_splits", [(16, 2, 128, 9), (14, 2, 64, 5)])
def test_attention_decode_of_many_unequal_sequences(ops, nh, kvh, d, n_splits):
    """More sequences than a warp has lanes (the kernel's plan walks them 32 at a time), lengths from one token to a
    few thousand, padding entries among them: long sequences are cut into several blocks, short ones into one."""
    g = torch.Generator().manual_seed(5)
    lengths = [int(v) for v in torch.randint(1, 400, (41,), generator=g)]
    lengths[3], lengths[17], lengths[40] = 2275, 1, 1500
    slots = list(range(41))[::-1]
    slots[5] = slots[33] = -1
    out, want = run_decode(ops, nh, kvh, d, lengths, 0, n_splits, slots=slots)
    assert max_err(out, want) <= 3e-2
    assert float(out[5].float().abs().max()) == 0.0 and float(out[33].float().abs().max()) == 0.0


def decode_plan_records(ops, lengths, kvh, nh, d, n_splits, slots=None, window=0):
    n = len(lengths)
    slots = slots if slots is not None else list(range(n))
    cu = torch.arange(n + 1, dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor([length - 1 for length in lengths], dtype=torch.int32, device=DEV)
    plan = ops.attention_decode_plan(cu, tok_pos, torch.tensor(slots, dtype=torch.int32, device=DEV), kvh, d, nh, n,
                                     window, n_splits, ops.DecodeScratch(DEV))
    table = plan.cpu().flatten()[:n].tolist()   # the plan's first part: every sequence's number of runs
    records = plan.cpu()[(n + 3) // 4:].tolist()
    at = 0
    for count in table:
        assert records[at][1] >> 16 == count
        at += count
    return records


def test_attention_decode_plan(ops):
    """Every sequence has its runs, numbered, one after another; together they fill the SMs at most once unless every
    sequence has only one; equal sequences get equal numbers; the rest of the grid is marked as empty."""
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    g = torch.Generator().manual_seed(11)
    ragged = [int(v) for v in torch.randint(64, 2300, (16,), generator=g)]
    cases = [([4096] * 8, 2, 14, 64, 8, None), ([4096] * 64, 2, 14, 64, 8, None), ([4096], 2, 14, 64, 8, None),
             (ragged, 2, 16, 128, 9, None), ([300, 5000, 1] + [70] * 40, 1, 40, 32, 10, [2, -1, 0] + list(range(3, 43)))]
    for lengths, kvh, nh, d, n_splits, slots in cases:
        records = decode_plan_records(ops, lengths, kvh, nh, d, n_splits, slots)
        slots = slots if slots is not None else list(range(len(lengths)))
        kvc = kvh * (-(-(nh // kvh) // 16))
        at, runs = 0, []
        for s, (length, slot) in enumerate(zip(lengths, slots)):
            n = records[at][1] >> 16
            assert 1 <= n <= n_splits
            for k in range(n):
                assert records[at + k] == [s, k | (n << 16), length if slot >= 0 else 0, slot], (lengths, s, k)
            pages = -(-length // 64) if slot >= 0 else 0
            assert n <= max(pages, 1) and (slot >= 0 or n == 1)
            runs.append(n)
            at += n
        assert all(r == [-1, 0, 0, -1] for r in records[at:])
        from qwenforge_b200.csrc import library
        room = int(library("attention_decode").qf_attention_decode_slots(d))   # blocks that the device holds at once
        assert room >= sms and sum(runs) * kvc <= room or all(n == 1 for n in runs), (lengths, runs)
        if len(set(zip(lengths, slots))) == 1 or len(set(lengths)) == 1 and min(slots) >= 0:
            assert len(set(runs)) == 1
    if sms == 148:   # the shapes that the split rule was measured at
        assert decode_plan_records(ops, [4096] * 8, 2, 14, 64, 8)[0][1] >> 16 == 8
        assert decode_plan_records(ops, [4096] * 64, 2, 14, 64, 8)[0][1] >> 16 == 1
        assert decode_plan_records(ops, [4096], 2, 14, 64, 8)[0][1] >> 16 == 8
        longest = max(range(16), key=lambda i: ragged[i])
        records = decode_plan_records(ops, ragged, 2, 16, 128, 9)
        assert max(r[1] >> 16 for r in records if r[0] == longest) >= 4   # the long one among short ones gets many blocks


@pytest.mark.parametrize("nh,kvh,d,lengths,n_out,n_splits,slots", [
    (14, 2, 64, [700, 64, 1, 2275, 130, 4000, 9, 333], 896, 8, None),     # the engine's shape at batch 8
    (16, 2, 128, [1200, 5], 2048, 5, None),
    (6, 3, 96, [300, 77, 1000], 272, 4, [2, -1, 0]),                      # a padding entry; outputs no multiple of 64
    (4, 4, 32, [50], 48, 1, None),                                        # one run only: partial results all the same
    (28, 4, 128, [600] * 16, 400, 3, None),                               # sixteen rows
])
def test_fold_project(ops, nh, kvh, d, lengths, n_out, n_splits, slots):
    """The decode attention stopped at its partial results, and the projection that folds them on its way in, against
    the attention kernel's own fold followed by a float64 product, and against the plain attention."""
    n = len(lengths)
    slots = slots if slots is not None else list(range(n))[::-1]
    site = FakeSite(n, max(lengths), kvh, d, torch.bfloat16, 31)
    for slot, length in zip(slots, lengths):
        if slot >= 0:
            fill_site(site, slot, length, 31 + slot, torch.bfloat16)
    g = torch.Generator().manual_seed(32)
    q = torch.randn(n, nh * d, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(n_out, nh * d, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    before = torch.randn(n, n_out, generator=g).to(DEV)
    cu = torch.arange(n + 1, dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor([length - 1 for length in lengths], dtype=torch.int32, device=DEV)
    slots_t = torch.tensor(slots, dtype=torch.int32, device=DEV)
    args = ops.KvSiteArgs(site.storage, site.table, kvh, d)
    e = err_word()
    assert ops.fold_project_takes(n, w, before, nh, d)
    scratch = ops.DecodeScratch(DEV)
    for _ in range(2):   # twice: nothing of the first call may be left in the scratch's way
        hidden = before.clone()
        plan = ops.attention_decode_plan(cu, tok_pos, slots_t, kvh, d, nh, n, 0, n_splits, scratch)
        ops.attention_decode(q, None, cu, tok_pos, slots_t, args, nh, n, d ** -0.5, 0, n_splits, scratch, e, plan, fold_later=True)
        ops.fold_project(plan, scratch, w, hidden, nh, d, n_splits)
    attended = torch.empty_like(q)
    ops.attention_decode(q, attended, cu, tok_pos, slots_t, args, nh, n, d ** -0.5, 0, n_splits, ops.DecodeScratch(DEV), e)
    assert int(e) == 0
    own = before.double() + attended.double() @ w.double().T
    bound = max(1.0, float(own.abs().max()))
    assert max_err(hidden, own) <= 1e-3 * bound
    plain = torch.empty_like(q)
    ref.attention_generic(q, plain, cu, tok_pos, slots_t, site, nh, n, 1, d ** -0.5, 0, None)
    assert max_err(hidden, before.double() + plain.double() @ w.double().T) <= 2e-2 * bound
    for r, slot in enumerate(slots):
        if slot < 0:
            assert torch.equal(hidden[r], before[r])


def test_fold_project_refuses_what_it_cannot_take(ops):
    hidden = torch.zeros(4, 100, device=DEV)
    w = torch.zeros(100, 4 * 64, dtype=torch.bfloat16, device=DEV)
    assert not ops.fold_project_takes(4, w, hidden, 4, 64)           # outputs no multiple of 16
    w = torch.zeros(96, 4 * 48, dtype=torch.bfloat16, device=DEV)
    assert not ops.fold_project_takes(4, w, torch.zeros(4, 96, device=DEV), 4, 48)    # a head is no multiple of 32 inputs
    w = torch.zeros(4096, 4 * 64, dtype=torch.bfloat16, device=DEV)
    assert not ops.fold_project_takes(4, w, torch.zeros(4, 4096, device=DEV), 4, 64)  # the slice does not fit shared memory
    w = torch.zeros(96, 4 * 64, dtype=torch.bfloat16, device=DEV)
    assert not ops.fold_project_takes(17, w, torch.zeros(17, 96, device=DEV), 4, 64)  # too many rows
    with pytest.raises(ops.KernelError, match="does not take"):
        ops.fold_project(torch.zeros(8, 4, dtype=torch.int32, device=DEV), ops.DecodeScratch(DEV), w,
                         torch.zeros(17, 96, device=DEV), 4, 64, 2)


def test_attention_decode_padding_and_far_key(ops):
    out, want = run_decode(ops, 4, 2, 64, [100, 50, 9], 0, 3, slots=[1, -1, 0])
    assert max_err(out, want) <= 3e-2 and float(out[1].float().abs().max()) == 0.0
    # one far key dominates: the output is its value, through every split
    nh, kvh, d, length = 2, 1, 64, 3000
    site = FakeSite(1, length, kvh, d, torch.bfloat16, 9)
    fill_site(site, 0, length, 3, torch.bfloat16)
    far = 70
    page, off = int(site.table[0, far // 64]), far % 64
    site.storage[page, 0, 0, off] = 0
    site.storage[page, 0, 0, off, 0] = 60.0
    q = torch.zeros(1, nh * d, dtype=torch.bfloat16, device=DEV)
    q[0, 0] = q[0, d] = 40.0
    out = torch.empty_like(q)
    cu = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    pos = torch.tensor([length - 1], dtype=torch.int32, device=DEV)
    slots = torch.tensor([0], dtype=torch.int32, device=DEV)
    ops.attention_decode(q, out, cu, pos, slots, ops.KvSiteArgs(site.storage, site.table, kvh, d), nh, 1, d ** -0.5, 0,
                         16, ops.DecodeScratch(DEV), err_word())
    value = site.storage[page, 1, 0, off]
    assert max_err(out[0, :d], value) < 2e-2 and max_err(out[0, d:], value) < 2e-2


# ------------------------------------------------------------------------------------------------ fused skinny products

def _normed_product(hidden, weight, eps, w):
    """rmsnorm(hidden) * weight times w^T with the kernel's one rounding of the operand: the rows enter the product
    as bfloat16(hidden * weight), and the sums are divided by the row's root mean square in float32 or better."""
    x = hidden.double()
    scaled = (x * weight.double()).to(torch.bfloat16).double()
    return (scaled @ w.double().T) * torch.rsqrt(x.square().mean(-1, keepdim=True) + eps)


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("n,k", [(896, 896), (50, 72), (1152, 4864), (17, 8),
                                 (5000, 1024), (2408, 544),      # more tiles than a wave: streamed through the ring
                                 (3584, 18944)])                 # and token rows too long to stay in shared memory
def test_skinny_gemm_plain_and_residual(ops, m, n, k):
    g = torch.Generator().manual_seed(20)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    b = torch.randn(n, generator=g).to(torch.bfloat16).to(DEV)
    want = x.double() @ w.double().T + b.double()
    bound = 2e-2 * max(1.0, float(want.abs().max()))
    for dtype in (torch.bfloat16, torch.float32):
        out = torch.empty(m, n, dtype=dtype, device=DEV)
        ops.skinny_gemm(ops.EPI_PLAIN, w, x=x, bias=b, out=out)
        assert max_err(out, want) <= (bound if dtype == torch.bfloat16 else bound / 20)
    hidden = torch.randn(m, n, generator=g).to(DEV)
    before = hidden.clone()
    ops.skinny_gemm(ops.EPI_RESIDUAL, w, x=x, residual=hidden)
    assert max_err(hidden, before.double() + x.double() @ w.double().T) <= bound / 20
    # the norm prologue
    stream = (torch.randn(m, k, generator=g) * 3).to(DEV)
    nw = (1 + 0.1 * torch.randn(k, generator=g)).to(torch.bfloat16).to(DEV)
    out = torch.empty(m, n, dtype=torch.float32, device=DEV)
    if k > 16384:
        # normalised rows of this length do not fit into shared memory beside the ring: refused, with the way out named
        with pytest.raises(ops.KernelError, match="use the unfused kernels"):
            ops.skinny_gemm(ops.EPI_PLAIN, w, hidden=stream, norm_weight=nw, eps=1e-5, out=out)
        return
    ops.skinny_gemm(ops.EPI_PLAIN, w, hidden=stream, norm_weight=nw, eps=1e-5, out=out)
    assert max_err(out, _normed_product(stream, nw, 1e-5, w)) <= bound / 10
    # a row's result does not depend on the other rows of the call
    if m > 1:
        one = torch.empty(1, n, dtype=torch.float32, device=DEV)
        ops.skinny_gemm(ops.EPI_PLAIN, w, hidden=stream[m - 1:], norm_weight=nw, eps=1e-5, out=one)
        assert torch.equal(one[0], out[m - 1])


@pytest.mark.parametrize("m,inter,k", [(2, 4864, 896), (8, 200, 120), (13, 24, 64),
                                       (16, 11008, 2048), (5, 18944, 3584)])   # streamed in several rounds
def test_skinny_gemm_swiglu(ops, m, inter, k):
    g = torch.Generator().manual_seed(21)
    stream = torch.randn(m, k, generator=g).to(DEV)
    nw = (1 + 0.1 * torch.randn(k, generator=g)).to(torch.bfloat16).to(DEV)
    w = (torch.randn(2 * inter, k, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    out = torch.empty(m, inter, dtype=torch.bfloat16, device=DEV)
    ops.skinny_gemm(ops.EPI_SWIGLU, w, hidden=stream, norm_weight=nw, eps=1e-6, out=out)
    gu = _normed_product(stream, nw, 1e-6, w)
    want = gu[:, :inter] * torch.sigmoid(gu[:, :inter]) * gu[:, inter:]
    assert max_err(out, want) <= 2e-2 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("m,nh,kvh,d,rotary,k", [(8, 14, 2, 64, True, 248), (3, 4, 4, 32, True, 248), (16, 8, 1, 128, False, 248),
                                                 (1, 6, 3, 96, True, 248),
                                                 (5, 28, 4, 128, True, 3584), (12, 40, 8, 64, True, 1056)])  # streamed through the ring
def test_skinny_gemm_qkv(ops, m, nh, kvh, d, rotary, k):
    """The fused projection + bias + rotation + cache write against the unfused references."""
    g = torch.Generator().manual_seed(22)
    stream = torch.randn(m, k, generator=g).to(DEV)
    nw = (1 + 0.1 * torch.randn(k, generator=g)).to(torch.bfloat16).to(DEV)
    n = (nh + 2 * kvh) * d
    w = (torch.randn(n, k, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    b = torch.randn(n, generator=g).to(torch.bfloat16).to(DEV)
    site_a, site_b = FakeSite(m, 400, kvh, d, torch.bfloat16), FakeSite(m, 400, kvh, d, torch.bfloat16)
    site_b.table = site_a.table
    positions = [(37 * i + 63) % 390 for i in range(m)]
    slots = [(m - 1 - i) if i != 1 else -1 for i in range(m)]
    tok_seq = torch.arange(m, dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor(positions, dtype=torch.int32, device=DEV)
    slots_t = torch.tensor(slots, dtype=torch.int32, device=DEV)
    inv_freq = (1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(DEV) if rotary else None
    q1 = torch.empty(m, nh * d, dtype=torch.bfloat16, device=DEV)
    e = err_word()
    ops.skinny_gemm(ops.EPI_QKV, w, hidden=stream, norm_weight=nw, eps=1e-6, bias=b,
                    qkv=dict(n_heads=nh, site=ops.KvSiteArgs(site_a.storage, site_a.table, kvh, d), inv_freq=inv_freq,
                             rot_dim=d if rotary else 0, tok_pos=tok_pos, tok_seq=tok_seq, slots=slots_t, q_out=q1,
                             write_cache=True, err=e))
    qkv = (_normed_product(stream, nw, 1e-6, w) + b.double()).to(torch.float32)
    q2 = torch.empty(m, nh * d, dtype=torch.float32, device=DEV)
    site_b.storage = site_b.storage.float()
    ref.rope_cache_write(qkv, tok_seq, tok_pos, slots_t, inv_freq, d if rotary else 0, nh, q2, site_b, True, None)
    assert int(e) == 0
    assert max_err(q1, q2) <= 3e-2 * max(1.0, float(q2.abs().max()))
    assert max_err(site_a.storage, site_b.storage) <= 3e-2 * max(1.0, float(site_b.storage.abs().max()))
    assert float(site_a.storage.float().abs().sum()) > 0


@pytest.mark.parametrize("m,n,k", [(16, 6400, 2048), (3, 5000, 3584), (9, 2400, 8192)])
def test_skinny_gemm_streams_many_tiles_in_rounds(ops, m, n, k):
    """More weight tiles than fit the SMs at once: blocks work through several batches with two weight buffers."""
    g = torch.Generator().manual_seed(24)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(n, k, generator=g) * 0.03).to(torch.bfloat16).to(DEV)
    want = x.double() @ w.double().T
    out = torch.empty(m, n, dtype=torch.float32, device=DEV)
    e = err_word()
    ops.skinny_gemm(ops.EPI_PLAIN, w, x=x, out=out, err=e)
    assert int(e) == 0 and max_err(out, want) <= 2e-3 * max(1.0, float(want.abs().max()))
    hidden = torch.randn(m, n, generator=g).to(DEV)
    before = hidden.clone()
    ops.skinny_gemm(ops.EPI_RESIDUAL, w, x=x, residual=hidden, err=e)
    assert int(e) == 0 and max_err(hidden, before.double() + want) <= 2e-3 * max(1.0, float(want.abs().max()))


def test_skinny_gemm_refuses_what_it_does_not_take(ops):
    w = torch.zeros(32, 20, dtype=torch.bfloat16, device=DEV)       # K not a multiple of 8
    x = torch.zeros(2, 20, dtype=torch.bfloat16, device=DEV)
    assert not ops.skinny_gemm_takes(2, w)
    with pytest.raises(ops.KernelError, match="not supported"):
        ops.skinny_gemm(ops.EPI_PLAIN, w, x=x, out=torch.empty(2, 32, dtype=torch.bfloat16, device=DEV))
    assert not ops.skinny_gemm_takes(17, torch.zeros(32, 64, dtype=torch.bfloat16, device=DEV))


def _layer_tail(ops, m, hidden_w, inter, nh, kvh, d, seed=50):
    """The four products that follow a decode step's attention, as descriptions: output projection into the stream,
    norm + gate/up + SwiGLU, down into the stream, norm + the next layer's QKV with rotation and cache write.
    Returns (products, state) where state holds every tensor that a run changes."""
    g = torch.Generator().manual_seed(seed)
    rnd = lambda *shape, scale=1.0: (torch.randn(*shape, generator=g) * scale)
    stream = rnd(m, hidden_w).to(DEV)
    attended = rnd(m, nh * d).to(torch.bfloat16).to(DEV)
    o_w = rnd(hidden_w, nh * d, scale=0.05).to(torch.bfloat16).to(DEV)
    gu_w = rnd(2 * inter, hidden_w, scale=0.05).to(torch.bfloat16).to(DEV)
    down_w = rnd(hidden_w, inter, scale=0.05).to(torch.bfloat16).to(DEV)
    qkv_w = rnd((nh + 2 * kvh) * d, hidden_w, scale=0.05).to(torch.bfloat16).to(DEV)
    qkv_b = rnd((nh + 2 * kvh) * d).to(torch.bfloat16).to(DEV)
    n1 = (1 + 0.1 * rnd(hidden_w)).to(torch.bfloat16).to(DEV)
    n2 = (1 + 0.1 * rnd(hidden_w)).to(torch.bfloat16).to(DEV)
    site = FakeSite(m, 400, kvh, d, torch.bfloat16)
    act = torch.zeros(m, inter, dtype=torch.bfloat16, device=DEV)
    q_out = torch.zeros(m, nh * d, dtype=torch.bfloat16, device=DEV)
    tok_seq = torch.arange(m, dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor([(37 * i + 63) % 390 for i in range(m)], dtype=torch.int32, device=DEV)
    slots = torch.tensor([(m - 1 - i) if i != 1 else -1 for i in range(m)], dtype=torch.int32, device=DEV)
    inv_freq = (1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(DEV)
    e = err_word()
    products = [
        ops.FusedProduct(ops.EPI_RESIDUAL, o_w, x=attended, residual=stream),
        ops.FusedProduct(ops.EPI_SWIGLU, gu_w, hidden=stream, norm_weight=n1, eps=1e-6, out=act),
        ops.FusedProduct(ops.EPI_RESIDUAL, down_w, x=act, residual=stream),
        ops.FusedProduct(ops.EPI_QKV, qkv_w, hidden=stream, norm_weight=n2, eps=1e-6, bias=qkv_b,
                         qkv=dict(n_heads=nh, site=ops.KvSiteArgs(site.storage, site.table, kvh, d), inv_freq=inv_freq,
                                  rot_dim=d, tok_pos=tok_pos, tok_seq=tok_seq, slots=slots, q_out=q_out, write_cache=True, err=e)),
    ]
    return products, dict(stream=stream, act=act, q_out=q_out, cache=site.storage, err=e)


@pytest.mark.parametrize("m,hidden_w,inter,nh,kvh,d", [(8, 896, 4864, 14, 2, 64), (1, 896, 4864, 14, 2, 64),
                                                      (3, 448, 608, 7, 1, 64), (5, 512, 736, 4, 2, 128),
                                                      (12, 448, 608, 7, 1, 64), (8, 2048, 11008, 16, 2, 128)])
def test_skinny_chain_equals_the_products_one_by_one(ops, m, hidden_w, inter, nh, kvh, d):
    """A decoder layer's products after attention as ONE persistent kernel against the same four run as separate
    kernels: the residual stream, the activations, the rotated queries and the cache pages. Twice over the same
    barrier words, bit for bit the same."""
    products, state = _layer_tail(ops, m, hidden_w, inter, nh, kvh, d)
    start = {k: v.clone() for k, v in state.items()}
    if not ops.skinny_chain_takes(products):
        assert m > 8 or hidden_w > 1024, "the chain kernel must take the small shapes"
        with pytest.raises(ops.KernelError, match="one by one"):
            ops.skinny_chain(products, torch.zeros(2, dtype=torch.int32, device=DEV), state["err"])
        return
    for product in products:
        product.run()
    want = {k: v.clone() for k, v in state.items()}
    assert int(state["err"]) == 0
    sync = torch.zeros(2, dtype=torch.int32, device=DEV)
    results = []
    for _ in range(2):
        for k, v in state.items():
            v.copy_(start[k])
        ops.skinny_chain(products, sync, state["err"])
        torch.cuda.synchronize()
        assert int(state["err"]) == 0
        results.append({k: v.clone() for k, v in state.items()})
    assert sync.tolist() == [0, 6]   # three barriers per launch, the arrival count back at zero
    for k in ("stream", "act", "q_out", "cache"):
        assert torch.equal(results[0][k], results[1][k]), k
        scale = max(1.0, float(want[k].float().abs().max()))
        assert max_err(results[0][k], want[k]) <= (2e-2 if want[k].dtype == torch.bfloat16 else 2e-3) * scale, k
    assert float(results[0]["cache"].float().abs().sum()) > 0
    # chains of one, two and three products
    for n in (1, 2, 3):
        for k, v in state.items():
            v.copy_(start[k])
        for product in products[:n]:
            product.run()
        want_n = state["stream"].clone(), state["act"].clone()
        for k, v in state.items():
            v.copy_(start[k])
        ops.skinny_chain(products[:n], sync, state["err"])
        assert max_err(state["stream"], want_n[0]) <= 2e-3 * max(1.0, float(want_n[0].abs().max()))
        assert max_err(state["act"], want_n[1]) <= 2e-2 * max(1.0, float(want_n[1].float().abs().max()))


# ------------------------------------------------------------------------------------------------ wide fused products

@pytest.mark.parametrize("m", [1, 17, 33, 64])
@pytest.mark.parametrize("n,k", [(896, 896), (200, 72), (896, 4864), (1152, 2048), (130, 8)])
def test_wide_gemm_plain_and_residual(ops, m, n, k):
    """Up to 64 token rows against the weights on tcgen05: plain (bf16 and float32, with a bias) and into the residual
    stream; K = 4864 against few tiles is split over a cluster."""
    g = torch.Generator().manual_seed(60)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    b = torch.randn(n, generator=g).to(torch.bfloat16).to(DEV)
    want = x.double() @ w.double().T
    scale = max(1.0, float(want.abs().max()))
    e = err_word()
    assert ops.wide_gemm_takes(ops.EPI_PLAIN, w, x=x, out=torch.empty(m, n, dtype=torch.float32, device=DEV))
    for dtype, tolerance in ((torch.float32, 2e-3), (torch.bfloat16, 2e-2)):
        out = torch.full((m, n), 7.0, dtype=dtype, device=DEV)
        ops.wide_gemm(ops.EPI_PLAIN, w, x=x, bias=b, out=out, err=e)
        assert int(e) == 0 and max_err(out, want + b.double()) <= tolerance * scale
    hidden = torch.randn(m, n, generator=g).to(DEV)
    before = hidden.clone()
    ops.wide_gemm(ops.EPI_RESIDUAL, w, x=x, residual=hidden, err=e)
    first = hidden.clone()
    assert int(e) == 0 and max_err(hidden, before.double() + want) <= 2e-3 * scale
    hidden.copy_(before)
    ops.wide_gemm(ops.EPI_RESIDUAL, w, x=x, residual=hidden, err=e)
    assert torch.equal(hidden, first)                       # the same sums in the same order, run after run
    if m > 1:                                               # and a row's result does not depend on the rows beside it
        alone = before[m - 1:].clone()
        ops.wide_gemm(ops.EPI_RESIDUAL, w, x=x[m - 1:], residual=alone, err=e)
        assert torch.equal(alone[0], first[m - 1])


@pytest.mark.parametrize("m,inter,k", [(64, 4864, 896), (17, 200, 120), (40, 64, 64), (33, 11008, 2048)])
def test_wide_gemm_swiglu(ops, m, inter, k):
    g = torch.Generator().manual_seed(61)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(2 * inter, k, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    out = torch.full((m, inter), 7.0, dtype=torch.bfloat16, device=DEV)
    e = err_word()
    ops.wide_gemm(ops.EPI_SWIGLU, w, x=x, out=out, err=e)
    gu = x.double() @ w.double().T
    want = gu[:, :inter] * torch.sigmoid(gu[:, :inter]) * gu[:, inter:]
    assert int(e) == 0 and max_err(out, want) <= 2e-2 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("m,nh,kvh,d,rotary,k", [(64, 14, 2, 64, True, 896), (17, 4, 4, 32, True, 248), (33, 8, 1, 128, False, 248),
                                                 (20, 6, 3, 16, True, 96), (48, 28, 4, 128, True, 3584)])
def test_wide_gemm_qkv(ops, m, nh, kvh, d, rotary, k):
    """The fused projection + bias + rotation + cache write for up to 64 tokens against the unfused references."""
    g = torch.Generator().manual_seed(62)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    n = (nh + 2 * kvh) * d
    w = (torch.randn(n, k, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    b = torch.randn(n, generator=g).to(torch.bfloat16).to(DEV)
    site_a, site_b = FakeSite(m, 400, kvh, d, torch.bfloat16), FakeSite(m, 400, kvh, d, torch.bfloat16)
    site_b.table = site_a.table
    positions = [(37 * i + 63) % 390 for i in range(m)]
    slots = [(m - 1 - i) if i != 1 else -1 for i in range(m)]
    tok_seq = torch.arange(m, dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor(positions, dtype=torch.int32, device=DEV)
    slots_t = torch.tensor(slots, dtype=torch.int32, device=DEV)
    inv_freq = (1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(DEV) if rotary else None
    q1 = torch.full((m, nh * d), 7.0, dtype=torch.bfloat16, device=DEV)
    e = err_word()
    ops.wide_gemm(ops.EPI_QKV, w, x=x, bias=b,
                  qkv=dict(n_heads=nh, site=ops.KvSiteArgs(site_a.storage, site_a.table, kvh, d), inv_freq=inv_freq,
                           rot_dim=d if rotary else 0, tok_pos=tok_pos, tok_seq=tok_seq, slots=slots_t, q_out=q1,
                           write_cache=True, err=e))
    qkv = (x.double() @ w.double().T + b.double()).to(torch.float32)
    q2 = torch.empty(m, nh * d, dtype=torch.float32, device=DEV)
    site_b.storage = site_b.storage.float()
    ref.rope_cache_write(qkv, tok_seq, tok_pos, slots_t, inv_freq, d if rotary else 0, nh, q2, site_b, True, None)
    assert int(e) == 0
    assert max_err(q1, q2) <= 3e-2 * max(1.0, float(q2.abs().max()))
    assert max_err(site_a.storage, site_b.storage) <= 3e-2 * max(1.0, float(site_b.storage.abs().max()))
    assert float(site_a.storage.float().abs().sum()) > 0


def test_wide_gemm_refuses_what_it_does_not_take(ops):
    w = torch.zeros(256, 64, dtype=torch.bfloat16, device=DEV)
    x = torch.zeros(65, 64, dtype=torch.bfloat16, device=DEV)     # more than 64 token rows
    out = torch.empty(65, 256, dtype=torch.bfloat16, device=DEV)
    assert not ops.wide_gemm_takes(ops.EPI_PLAIN, w, x=x, out=out)
    with pytest.raises(ops.KernelError, match="not supported"):
        ops.wide_gemm(ops.EPI_PLAIN, w, x=x, out=out)
    w96 = torch.zeros(5 * 96, 64, dtype=torch.bfloat16, device=DEV)   # a head size that does not divide 128
    site = FakeSite(4, 64, 1, 96, torch.bfloat16)
    args = dict(x=x[:4], qkv=dict(n_heads=3, site=ops.KvSiteArgs(site.storage, site.table, 1, 96), inv_freq=None, rot_dim=0,
                                  tok_pos=torch.zeros(4, dtype=torch.int32, device=DEV), tok_seq=torch.zeros(4, dtype=torch.int32, device=DEV),
                                  slots=torch.zeros(1, dtype=torch.int32, device=DEV),
                                  q_out=torch.empty(4, 3 * 96, dtype=torch.bfloat16, device=DEV), write_cache=False, err=err_word()))
    assert not ops.wide_gemm_takes(ops.EPI_QKV, w96, **args)


def test_residual_add(ops):
    g = torch.Generator().manual_seed(23)
    h = torch.randn(5, 77, generator=g).to(DEV)
    d = torch.randn(5, 77, generator=g).to(torch.bfloat16).to(DEV)
    want = h + d.float()
    ops.residual_add(h, d)
    assert torch.equal(h, want)


@pytest.mark.parametrize("dtype", DTYPES)
def test_rope_cache_write_adds_the_bias_first(ops, dtype):
    g = torch.Generator().manual_seed(30)
    nh, kvh, d, n = 3, 1, 32, 5
    site_a, site_b = FakeSite(1, 64, kvh, d, dtype), FakeSite(1, 64, kvh, d, dtype)
    site_b.table = site_a.table
    qkv = torch.randn(n, (nh + 2 * kvh) * d, generator=g).to(dtype).to(DEV)
    bias = torch.randn((nh + 2 * kvh) * d, generator=g).to(dtype).to(DEV)
    tok_seq = torch.zeros(n, dtype=torch.int32, device=DEV)
    tok_pos = torch.arange(7, 7 + n, dtype=torch.int32, device=DEV)
    slots = torch.zeros(1, dtype=torch.int32, device=DEV)
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, 16, 2, dtype=torch.float32) / 16))).to(DEV)   # half of the head rotates
    q1 = torch.empty(n, nh * d, dtype=dtype, device=DEV)
    q2 = torch.empty_like(q1)
    e = err_word()
    ops.rope_cache_write(qkv, tok_seq, tok_pos, slots, inv_freq, 16, nh, q1, ops.KvSiteArgs(site_a.storage, site_a.table, kvh, d),
                         True, e, bias=bias)
    ref.rope_cache_write(qkv, tok_seq, tok_pos, slots, inv_freq, 16, nh, q2, site_b, True, None, bias=bias)
    assert int(e) == 0 and max_err(q1, q2) <= tol(dtype) * 8 and max_err(site_a.storage, site_b.storage) <= tol(dtype) * 8


def test_linear_bf16_matches_a_plain_product(ops):
    g = torch.Generator().manual_seed(31)
    for m, n, k in ((1, 8, 16), (70, 200, 120), (2048, 1152, 896)):
        x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
        w = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
        b = torch.randn(n, generator=g).to(torch.bfloat16).to(DEV)
        want = x.double() @ w.double().T
        assert max_err(ops.linear(x, w), want) <= 2e-2 * max(1.0, float(want.abs().max()))
        assert max_err(ops.linear(x, w, out_dtype=torch.float32), want) <= 2e-3 * max(1.0, float(want.abs().max()))
        assert ops.linear(x, w, out_dtype=torch.float32).dtype == torch.float32
        assert max_err(ops.linear(x, w, b), want + b.double()) <= 3e-2 * max(1.0, float(want.abs().max()))
        wide = torch.randn(m, k + 8, generator=g).to(torch.bfloat16).to(DEV)   # strided rows
        assert max_err(ops.linear(wide[:, :k], w), wide[:, :k].double() @ w.double().T) <= 2e-2 * max(1.0, float(want.abs().max()))


# ------------------------------------------------------------------------------------------------ tcgen05 products

# the last three have tiles for every SM and more: the persistent kernel, with ragged last tiles in every direction
@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (200, 1152, 896), (2048, 896, 4864), (130, 136, 72), (1, 8, 8),
                                   (2048, 9728, 896), (1999, 5000, 264), (4100, 2568, 72)])
def test_tc_gemm_plain(ops, m, n, k):
    g = torch.Generator().manual_seed(40)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    out = torch.full((m, n), 7.0, dtype=torch.bfloat16, device=DEV)
    e = err_word()
    ops.tc_gemm(ops.TC_PLAIN, x, w, out, e)
    want = x.double() @ w.double().T
    assert int(e) == 0 and max_err(out, want) <= 2e-2 * max(1.0, float(want.abs().max()))
    assert ops.tc_gemm_is_persistent(ops.TC_PLAIN, m, n) == (-(-m // 128) * -(-n // 256) >= ops.sm_count(DEV))
    assert ops.tc_gemm_is_persistent(ops.TC_PLAIN, m, n) == (m >= 1999 and n > 1000)   # the cases meant for it reach it


# the last three run in the persistent kernel (ragged last tiles of rows and of features, a K that is no multiple of 64)
@pytest.mark.parametrize("m,inter,k", [(128, 64, 64), (300, 200, 896), (70, 72, 120), (2048, 4864, 896), (1999, 2504, 264),
                                       (700, 3400, 1000)])
def test_tc_gemm_swiglu(ops, m, inter, k):
    g = torch.Generator().manual_seed(41)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(2 * inter, k, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    out = torch.full((m, inter), 7.0, dtype=torch.bfloat16, device=DEV)
    e = err_word()
    ops.tc_gemm(ops.TC_SWIGLU, x, w, out, e)
    gu = x.double() @ w.double().T
    want = gu[:, :inter] * torch.sigmoid(gu[:, :inter]) * gu[:, inter:]
    assert int(e) == 0 and max_err(out, want) <= 2e-2 * max(1.0, float(want.abs().max()))
    assert ops.tc_gemm_is_persistent(ops.TC_SWIGLU, m, 2 * inter) == (-(-m // 128) * -(-inter // 128) >= ops.sm_count(DEV))
    assert ops.tc_gemm_is_persistent(ops.TC_SWIGLU, m, 2 * inter) == (m >= 700)   # the cases meant for it reach it


@pytest.mark.parametrize("q_lens,nh,kvh,d,k,rotary,with_bias", [
    ([300, 1, 70], 7, 1, 64, 448, True, True),        # three sequences, a padding entry, ragged last tiles of rows and of heads
    ([640], 14, 2, 64, 896, True, True),              # Qwen2.5-0.5B's heads
    ([130, 64], 4, 2, 128, 264, True, False),         # one head per tile, K no multiple of 64
    ([200], 3, 3, 32, 120, True, True),               # four heads per tile
    ([150], 5, 1, 64, 72, False, True),               # no rotation
])
def test_tc_gemm_qkv(ops, q_lens, nh, kvh, d, k, rotary, with_bias):
    """The query/key/value product with bias, rotation and cache write in its epilogue, against the float64 product put
    through the plain rotation and cache write; the cache untouched where nothing is to be written."""
    g = torch.Generator().manual_seed(44)
    n, n_seqs = sum(q_lens), len(q_lens)
    starts = [0, 63, 60][:n_seqs]
    slots = [2, -1, 0][:n_seqs] if n_seqs == 3 else list(range(n_seqs))[::-1]
    site_a = FakeSite(3, 1024, kvh, d, torch.bfloat16)
    site_b = FakeSite(3, 1024, kvh, d, torch.bfloat16)
    site_b.table = site_a.table
    x = torch.randn(n, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn((nh + 2 * kvh) * d, k, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    bias = torch.randn((nh + 2 * kvh) * d, generator=g).to(torch.bfloat16).to(DEV) if with_bias else None
    tok_seq = torch.tensor(sum(([i] * q for i, q in enumerate(q_lens)), []), dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor(sum((list(range(s, s + q)) for s, q in zip(starts, q_lens)), []), dtype=torch.int32, device=DEV)
    slots_t = torch.tensor(slots, dtype=torch.int32, device=DEV)
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(DEV) if rotary else None
    angles = ops.rope_table(tok_pos, inv_freq) if rotary else None
    if rotary:
        want_angle = tok_pos.float().unsqueeze(-1) * inv_freq
        assert max_err(angles[..., 0], want_angle.double().cos()) < 1e-6 and max_err(angles[..., 1], want_angle.double().sin()) < 1e-6
    q1 = torch.full((n, nh * d), 7.0, dtype=torch.bfloat16, device=DEV)
    q2 = torch.empty_like(q1)
    e = err_word()
    args = ops.KvSiteArgs(site_a.storage, site_a.table, kvh, d)
    assert ops.tc_gemm_qkv_takes(x, w, d)
    ops.tc_gemm_qkv(x, w, bias, angles, tok_seq, tok_pos, slots_t, nh, q1, args, True, e)
    product = x.double() @ w.double().T
    ref.rope_cache_write(product, tok_seq, tok_pos, slots_t, inv_freq, d if rotary else 0, nh, q2, site_b, True, None, bias=bias)
    scale = max(1.0, float(product.abs().max()))
    assert int(e) == 0
    assert max_err(q1, q2) <= 2e-2 * scale
    assert max_err(site_a.storage, site_b.storage) <= 2e-2 * scale and float(site_a.storage.float().abs().sum()) > 0
    before = site_a.storage.clone()
    ops.tc_gemm_qkv(x, w, bias, angles, tok_seq, tok_pos, slots_t, nh, q1, args, False, e)   # without the write flag
    assert int(e) == 0 and torch.equal(before, site_a.storage) and max_err(q1, q2) <= 2e-2 * scale


def test_tc_gemm_refuses_misaligned_shapes(ops):
    x = torch.zeros(4, 20, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(8, 20, dtype=torch.bfloat16, device=DEV)
    assert not ops.tc_gemm_takes(x, w)
    with pytest.raises(ops.KernelError):
        ops.tc_gemm(ops.TC_PLAIN, x, w, torch.zeros(4, 8, dtype=torch.bfloat16, device=DEV))
