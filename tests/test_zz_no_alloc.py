"""The decode attention entry point that allocates nothing (`qf_attention_decode_noalloc`).

Some callers of the kernel library cannot allocate device memory when they need attention: a host program that
handed out all GPU memory at start-up, or a step that must not risk an allocation blocking or failing halfway.
For them the library has one entry point whose scratch is an array inside the library itself. This test calls it
the way such a caller would, through the exported C symbol, and checks it against the ordinary entry point
(which takes scratch from the caller) within the tolerance of the other attention tests, on two calls in a row
with different inputs: the second call meets the scratch as the first one left it. The file is named so that
pytest collects it last.
"""
import ctypes

import pytest
import torch

from tests.helpers import max_err
from tests.test_kernels_gpu import FakeSite, fill_site

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _call(lib, q, out, cu, tok_pos, slots, site, kvh, d, nh, n, window, n_splits, err):
    P, I, F, LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
    fn = lib.qf_attention_decode_noalloc
    fn.restype = ctypes.c_int
    return fn(P(q.data_ptr()), P(out.data_ptr()), P(cu.data_ptr()), P(tok_pos.data_ptr()), P(slots.data_ptr()),
              P(site.storage.data_ptr()), P(site.table.data_ptr()), LL(site.storage.stride(0)), I(site.table.stride(0)),
              I(kvh), I(d), I(nh), I(n), F(d ** -0.5), I(window), I(n_splits), P(err.data_ptr()),
              P(torch.cuda.current_stream().cuda_stream))


def test_no_alloc_entry_point_matches_the_ordinary_one_twice():
    from qwenforge_b200 import ops
    from qwenforge_b200.csrc import library
    lib = library("attention_decode")
    message = lib.qf_attention_decode_noalloc_error
    message.restype = ctypes.c_char_p
    nh, kvh, d = 14, 2, 64
    for round_, (lengths, n_splits, window) in enumerate([([700, 64, 1, 333], 5, 0), ([129, 1000], 16, 300)]):
        n = len(lengths)
        site = FakeSite(n, max(lengths), kvh, d, torch.bfloat16, 40 + round_)
        for slot, length in enumerate(lengths):
            fill_site(site, slot, length, 50 + round_ + slot, torch.bfloat16)
        g = torch.Generator().manual_seed(60 + round_)
        q = torch.randn(n, nh * d, generator=g).to(torch.bfloat16).to(DEV)
        cu = torch.arange(n + 1, dtype=torch.int32, device=DEV)
        tok_pos = torch.tensor([length - 1 for length in lengths], dtype=torch.int32, device=DEV)
        slots = torch.arange(n, dtype=torch.int32, device=DEV)
        err = torch.zeros(1, dtype=torch.int32, device=DEV)
        want = torch.empty_like(q)
        ops.attention_decode(q, want, cu, tok_pos, slots, ops.KvSiteArgs(site.storage, site.table, kvh, d), nh, n,
                             d ** -0.5, window, n_splits, ops.DecodeScratch(DEV), err)
        got = torch.full_like(q, 7.0)
        before = torch.cuda.memory_allocated()
        code = _call(lib, q, got, cu, tok_pos, slots, site, kvh, d, nh, n, window, n_splits, err)
        torch.cuda.synchronize()
        assert code == 0, message().decode()
        assert torch.cuda.memory_allocated() == before
        assert int(err) == 0
        assert max_err(got, want) <= 3e-2
        assert torch.equal(got, want)   # the same kernel on the same inputs: bit for bit


def test_no_alloc_entry_point_refuses_what_exceeds_its_scratch():
    from qwenforge_b200.csrc import library
    lib = library("attention_decode")
    message = lib.qf_attention_decode_noalloc_error
    message.restype = ctypes.c_char_p
    nh, kvh, d, n = 64, 8, 64, 64          # 64 * 64 * 4 splits = 16384 rows of partial results
    site = FakeSite(1, 64, kvh, d, torch.bfloat16, 1)
    q = torch.zeros(n, nh * d, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros_like(q)
    cu = torch.arange(n + 1, dtype=torch.int32, device=DEV)
    zeros = torch.zeros(n, dtype=torch.int32, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    code = _call(lib, q, out, cu, zeros, zeros, site, kvh, d, nh, n, 0, 4, err)
    assert code == -2 and b"limit 8192" in message()
    torch.cuda.synchronize()
