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


def _case(seed, lens, nq, nkv, hd, rows=None):
    """``rows``: the token index of each sequence's query inside a larger packed buffer (cu_q);
    None: one row per sequence, in order."""
    g = torch.Generator().manual_seed(seed)
    B = len(lens)
    n_rows = B if rows is None else max(rows) + 2
    pages_each = [(n + 63) // 64 for n in lens]
    n_pages = sum(pages_each) + 2
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((B, max(pages_each) + 1), -1, dtype=torch.int32)
    for b, p in enumerate(pages_each):
        for j in range(p):
            table[b, j] = order.pop()
    kc = torch.randn((n_pages, nkv, 64, hd), generator=g).bfloat16()
    vc = torch.randn((n_pages, nkv, 64, hd), generator=g).bfloat16()
    q = torch.randn((n_rows, nq * hd), generator=g).bfloat16()
    cu_q = torch.arange(B + 1, dtype=torch.int32) if rows is None else torch.tensor(list(rows) + [n_rows], dtype=torch.int32)
    ints = dict(table=table, seq_slot=torch.arange(B, dtype=torch.int32),
                cu_q=cu_q, kv_len=torch.tensor(lens, dtype=torch.int32))
    return q.to(DEV), kc.to(DEV), vc.to(DEV), {k: v.to(DEV) for k, v in ints.items()}


def _float64(q, kc, vc, d, lens, nq, nkv, hd, window):
    """Softmax attention of each sequence's one query over its own keys, gathered page by page, in
    float64 on the host: head h reads key/value head h // (nq / nkv); the query sits at the last
    position and, with a window, sees the last ``window`` keys only."""
    q, kc, vc = q.double().cpu(), kc.double().cpu(), vc.double().cpu()
    table, cu_q = d["table"].cpu(), d["cu_q"].cpu()
    out = torch.zeros_like(q)
    for b, n in enumerate(lens):
        pages = table[b, :(n + 63) // 64].long()
        k = kc[pages].permute(1, 0, 2, 3).reshape(nkv, -1, hd)[:, :n]
        v = vc[pages].permute(1, 0, 2, 3).reshape(nkv, -1, hd)[:, :n]
        lo = max(0, n - window) if window else 0
        t = int(cu_q[b])
        for h in range(nq):
            kv = h // (nq // nkv)
            s = (k[kv, lo:] @ q[t, h * hd:(h + 1) * hd]) / math.sqrt(hd)
            out[t, h * hd:(h + 1) * hd] = torch.softmax(s, dim=0) @ v[kv, lo:]
    return out


def _both_ways(fn, seed, lens, nq, nkv, hd, window=0, rows=None):
    from rocml_b200 import kernels
    q, kc, vc, d = _case(seed, lens, nq, nkv, hd, rows)
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
    used = d["cu_q"][:B].long()
    got, want = got[used], want[used]                  # rows that belong to no sequence stay untouched
    assert torch.isfinite(got.float()).all()
    err = (got.float() - want.float()).abs().max().item()
    assert err < 2e-2, err          # the tolerance of the attention tests; in fact the two agree exactly
    ref = _float64(q, kc, vc, d, lens, nq, nkv, hd, window)[used.cpu()]
    err64 = (got.double().cpu() - ref).abs().max().item()
    assert err64 < 2e-2, err64      # and both are right, not only alike
    return got, want


def test_static_scratch_entry_point_matches_the_ordinary_one_twice_in_a_row():
    fn = _symbol()
    a, wa = _both_ways(fn, 1, [700, 1, 129, 64, 300], 32, 8, 128)
    b, wb = _both_ways(fn, 2, [90, 513, 2], 8, 2, 64, window=100)      # other sizes meet the first call's leftovers
    c, wc = _both_ways(fn, 1, [700, 1, 129, 64, 300], 32, 8, 128)      # and the first case again
    assert torch.equal(a, c) and torch.equal(a, wa) and torch.equal(b, wb)


def test_static_scratch_entry_point_when_the_partial_results_go_through_the_array():
    """Up to 16 chunks the kernel's blocks merge through shared memory and the array is not touched.
    Beyond that the partial results, their maxima and sums and the arrival counters all live in the
    array: sequences of 18 and 21 chunks, twice in a row with different shapes, so that the second
    call finds the first call's partial results and counters there."""
    fn = _symbol()
    a, wa = _both_ways(fn, 5, [1100, 70, 1], 8, 2, 64)
    b, wb = _both_ways(fn, 6, [300, 1290, 1030, 64], 32, 8, 128, window=0)
    c, wc = _both_ways(fn, 5, [1100, 70, 1], 8, 2, 64)
    assert torch.equal(a, c) and torch.equal(a, wa) and torch.equal(b, wb)


def test_static_scratch_entry_point_with_queries_taken_from_a_larger_buffer():
    """cu_q names rows far beyond the number of sequences (the queries are three rows of a packed
    buffer of 41): the array is indexed by the sequence's place in the batch, so nothing is written
    outside the limits that were checked."""
    fn = _symbol()
    _both_ways(fn, 7, [1100, 200, 65], 8, 2, 64, rows=[39, 3, 17])
    _both_ways(fn, 8, [500, 130], 32, 8, 128, rows=[20, 7])         # the cluster path, same indexing of q and out


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    fn = _symbol()
    q = torch.zeros((1, 128), dtype=torch.bfloat16, device=DEV)
    z = torch.zeros(4, dtype=torch.int32, device=DEV)
    # 256 sequences x 64 heads x 512 chunks x 128 is far beyond 4 Mi floats; nothing may be launched or read
    rc = fn(q.data_ptr(), 128, q.data_ptr(), q.data_ptr(), z.data_ptr(), 1, z.data_ptr(), z.data_ptr(), z.data_ptr(),
            256, 64, 8, 128, 0.1, 0, 512, q.data_ptr(), 128, torch.cuda.current_stream().cuda_stream)
    assert rc == RB_ERR_SCRATCH_LIMIT
    torch.cuda.synchronize()
