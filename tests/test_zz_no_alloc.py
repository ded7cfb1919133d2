"""The entry point for callers that cannot allocate, called the way such a caller calls it: through
its exported C symbol, with nothing but pointers to its own inputs and outputs.

Its result must equal that of the ordinary entry point (which takes the work space from the caller)
on two calls in a row with different inputs: the second call meets whatever the first left in the
shared array.  Sizes beyond the array are refused before anything is launched.  The file is named so
that pytest collects it last.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
RB_ERR_SCRATCH_LIMIT = 10006


def _symbol():
    from rocml_b200.csrc import build
    lib = ctypes.CDLL(build.build(verbose=False))
    fn = lib.rb_attention_decode_static
    vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [vp, i, vp, vp, vp, i, vp, vp, vp, i, i, i, i, f, i, i, vp, i, vp]
    fn.restype = i
    return fn


def _case(seed, lens, nq, nkv, hd):
    g = torch.Generator().manual_seed(seed)
    B = len(lens)
    pages_each = [(n + 63) // 64 for n in lens]
    n_pages = sum(pages_each) + 2
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((B, max(pages_each) + 1), -1, dtype=torch.int32)
    for b, p in enumerate(pages_each):
        for j in range(p):
            table[b, j] = order.pop()
    kc = torch.randn((n_pages, nkv, 64, hd), generator=g).bfloat16()
    vc = torch.randn((n_pages, nkv, 64, hd), generator=g).bfloat16()
    q = torch.randn((B, nq * hd), generator=g).bfloat16()
    ints = dict(table=table, seq_slot=torch.arange(B, dtype=torch.int32),
                cu_q=torch.arange(B + 1, dtype=torch.int32), kv_len=torch.tensor(lens, dtype=torch.int32))
    return q.to(DEV), kc.to(DEV), vc.to(DEV), {k: v.to(DEV) for k, v in ints.items()}


def _both_ways(fn, seed, lens, nq, nkv, hd, window=0):
    from rocml_b200 import kernels
    q, kc, vc, d = _case(seed, lens, nq, nkv, hd)
    B = len(lens)
    scale = 1.0 / math.sqrt(hd)
    n_chunks = (max(lens) + 63) // 64
    # the ordinary entry point: the caller brings the work space
    want = torch.full_like(q, float("nan"))
    acc = torch.empty((B, nq, n_chunks, hd), dtype=torch.float32, device=DEV)
    ml = torch.empty((B, nq, n_chunks, 2), dtype=torch.float32, device=DEV)
    assert kernels.attention_decode(q, want, kc, vc, d["table"], d["seq_slot"], d["cu_q"], d["kv_len"], B, nq, nkv,
                                    hd, scale, window, n_chunks, acc, ml)
    # the entry point that allocates nothing
    got = torch.full_like(q, float("nan"))
    stream = torch.cuda.current_stream().cuda_stream
    held = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    rc = fn(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), d["table"].data_ptr(), d["table"].shape[1],
            d["seq_slot"].data_ptr(), d["cu_q"].data_ptr(), d["kv_len"].data_ptr(), B, nq, nkv, hd, scale, window,
            n_chunks, got.data_ptr(), got.stride(0), stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert (torch.cuda.memory_allocated(), torch.cuda.memory_reserved()) == held   # it took nothing from the allocator
    assert torch.isfinite(got.float()).all()
    err = (got.float() - want.float()).abs().max().item()
    assert err < 2e-2, err          # the tolerance of the attention tests; in fact the two agree exactly
    return got, want


def test_static_scratch_entry_point_matches_the_ordinary_one_twice_in_a_row():
    fn = _symbol()
    a, wa = _both_ways(fn, 1, [700, 1, 129, 64, 300], 32, 8, 128)
    b, wb = _both_ways(fn, 2, [90, 513, 2], 8, 2, 64, window=100)      # other sizes meet the first call's leftovers
    c, wc = _both_ways(fn, 1, [700, 1, 129, 64, 300], 32, 8, 128)      # and the first case again
    assert torch.equal(a, c) and torch.equal(a, wa) and torch.equal(b, wb)


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    fn = _symbol()
    q = torch.zeros((1, 128), dtype=torch.bfloat16, device=DEV)
    z = torch.zeros(4, dtype=torch.int32, device=DEV)
    # 256 sequences x 64 heads x 512 chunks x 128 is far beyond 4 Mi floats; nothing may be launched or read
    rc = fn(q.data_ptr(), 128, q.data_ptr(), q.data_ptr(), z.data_ptr(), 1, z.data_ptr(), z.data_ptr(), z.data_ptr(),
            256, 64, 8, 128, 0.1, 0, 512, q.data_ptr(), 128, torch.cuda.current_stream().cuda_stream)
    assert rc == RB_ERR_SCRATCH_LIMIT
    torch.cuda.synchronize()
