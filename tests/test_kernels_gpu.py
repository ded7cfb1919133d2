"""Each CUDA kernel alone against a plain torch reference of the same operation (float64 on the
CPU), at sizes other than the engine's tiny models use."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def rnd(shape, seed, dtype=torch.float32, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


# ---- matrix products ----------------------------------------------------------------------------

GEMM_SHAPES = [(1, 300, 64), (5, 128, 72), (16, 1000, 512), (17, 96, 208), (64, 4096, 1024),
               (100, 515, 1024), (128, 256, 2048), (129, 777, 264), (300, 256, 4096), (1500, 1024, 512)]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_tcgen05(M, N, K, out_dtype):
    from rocml_b200 import kernels
    x = rnd((M, K), 1, torch.bfloat16).to(DEV)
    w = rnd((N, K), 2, torch.bfloat16).to(DEV)
    bias = rnd((N,), 3).to(DEV)
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    assert kernels.gemm_tcgen05(x, w, out, bias)
    kernels.check_status(DEV)
    want = x.cpu().double() @ w.cpu().double().t() + bias.cpu().double()
    tol = 2 ** -8 if out_dtype == torch.bfloat16 else 1e-5
    scale = (x.cpu().double().abs() @ w.cpu().double().abs().t()).clamp_min(1.0)
    err = ((out.cpu().double() - want).abs() / scale).max().item()
    assert err < tol, err


@pytest.mark.parametrize("M,N,K,S", [(1, 4096, 4096, 4), (8, 520, 1024, 3), (64, 256, 12288, 8), (33, 1000, 200, 2)])
def test_gemm_tcgen05_split_k(M, N, K, S):
    from rocml_b200 import kernels
    x = rnd((M, K), 4, torch.bfloat16).to(DEV)
    w = rnd((N, K), 5, torch.bfloat16).to(DEV)
    bias = rnd((N,), 6).to(DEV)
    out = torch.full((S, M, N), float("nan"), dtype=torch.float32, device=DEV)
    assert kernels.gemm_tcgen05(x, w, out, bias)
    kernels.check_status(DEV)
    want = x.cpu().double() @ w.cpu().double().t() + bias.cpu().double()
    scale = (x.cpu().double().abs() @ w.cpu().double().abs().t()).clamp_min(1.0)
    err = ((out.cpu().double().sum(0) - want).abs() / scale).max().item()
    assert err < 1e-5, err


@pytest.mark.parametrize("M,I,K", [(1, 208, 96), (8, 12288, 512), (64, 320, 128), (200, 4096, 1024), (2048, 1024, 256)])
def test_gemm_tcgen05_gated_epilogue(M, I, K):
    """gate and up rows interleaved in blocks of 16; the product's epilogue gives silu(gate) * up."""
    from rocml_b200 import kernels
    x = rnd((M, K), 1, torch.bfloat16).to(DEV)
    wg, wu = rnd((I, K), 2, torch.bfloat16, 0.2), rnd((I, K), 3, torch.bfloat16, 0.2)
    bg, bu = rnd((I,), 4), rnd((I,), 5)
    mix = lambda g, u: torch.stack([g.reshape(I // 16, 16, *g.shape[1:]), u.reshape(I // 16, 16, *u.shape[1:])], 1).reshape(2 * I, *g.shape[1:])
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert kernels.gemm_tcgen05(x, mix(wg, wu).contiguous().to(DEV), out, mix(bg, bu).contiguous().to(DEV), gated=True)
    kernels.check_status(DEV)
    xd = x.cpu().double()
    g = xd @ wg.double().t() + bg.double()
    u = xd @ wu.double().t() + bu.double()
    want = g / (1 + torch.exp(-g)) * u
    err = ((out.cpu().double() - want).abs() / want.abs().clamp_min(1.0)).max().item()
    assert err < 2 ** -7, err


@pytest.mark.parametrize("M,I,K", [(1, 208, 256), (8, 12288, 512), (32, 320, 1024), (17, 4096, 4096), (16, 48, 136)])
def test_gemm_tcgen05_gated_pair_of_blocks(M, I, K):
    """Few rows, the sum over K in two halves by the two blocks of a cluster: the second hands its
    accumulator to the first through shared memory, the first writes silu(gate) * up."""
    from rocml_b200 import kernels
    x = rnd((M, K), 1, torch.bfloat16).to(DEV)
    wg, wu = rnd((I, K), 2, torch.bfloat16, 0.2), rnd((I, K), 3, torch.bfloat16, 0.2)
    bg, bu = rnd((I,), 4), rnd((I,), 5)
    mix = lambda g, u: torch.stack([g.reshape(I // 16, 16, *g.shape[1:]), u.reshape(I // 16, 16, *u.shape[1:])], 1).reshape(2 * I, *g.shape[1:])
    w, b = mix(wg, wu).contiguous().to(DEV), mix(bg, bu).contiguous().to(DEV)
    xd = x.cpu().double()
    g = xd @ wg.double().t() + bg.double()
    u = xd @ wu.double().t() + bu.double()
    want = g / (1 + torch.exp(-g)) * u
    for _ in range(2):
        out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
        assert kernels.gemm_tcgen05_gated_pair(x, w, out, b)
        kernels.check_status(DEV)
        err = ((out.cpu().double() - want).abs() / want.abs().clamp_min(1.0)).max().item()
        assert err < 2 ** -7, err
    assert kernels.gemm_tcgen05_gated_pair(rnd((40, K), 1, torch.bfloat16).to(DEV), w,
                                           torch.empty((40, I), dtype=torch.bfloat16, device=DEV)) is False


@pytest.mark.parametrize("M,N,K,S,wdt", [(1, 4096, 4096, 8, torch.bfloat16), (8, 520, 1024, 4, torch.float32),
                                         (16, 256, 12288, 16, torch.bfloat16), (3, 1000, 512, 8, torch.float32),
                                         (33, 520, 1024, 8, torch.bfloat16), (64, 4096, 512, 8, torch.float32),
                                         (20, 300, 2048, 16, torch.bfloat16)])
def test_gemm_tcgen05_adds_into_the_residual_stream(M, N, K, S, wdt):
    """The product of few rows, added to the float32 residual by the blocks of a cluster, with what the
    following norm needs: residual * weight in bfloat16 and the rows' sums of squares in shares."""
    from rocml_b200 import kernels
    x = rnd((M, K), 4, torch.bfloat16).to(DEV)
    w = rnd((N, K), 5, torch.bfloat16, 0.05).to(DEV)
    bias = rnd((N,), 6).to(DEV)
    nw = (1 + 0.1 * rnd((N,), 7)).to(wdt).to(DEV)
    resid0 = rnd((M, N), 8)
    want = resid0.double() + x.cpu().double() @ w.cpu().double().t() + bias.cpu().double()
    for _ in range(2):
        resid = resid0.clone().to(DEV)
        xhat = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        sumsq = torch.full((((N + 127) // 128) * S, M), float("nan"), dtype=torch.float32, device=DEV)
        assert kernels.gemm_tcgen05_residual(x, w, resid, S, bias, nw, xhat, sumsq)
        kernels.check_status(DEV)
        scale = want.abs().clamp_min(1.0)
        assert ((resid.cpu().double() - want).abs() / scale).max().item() < 1e-5
        assert ((xhat.cpu().double() - want * nw.cpu().double()).abs() / scale).max().item() < 2 ** -7
        got_ss = sumsq.cpu().double().sum(0)
        assert ((got_ss - (want ** 2).sum(1)).abs() / (want ** 2).sum(1)).max().item() < 1e-5
    # only the addition, nothing for a norm
    resid = resid0.clone().to(DEV)
    assert kernels.gemm_tcgen05_residual(x, w, resid, S, bias)
    assert ((resid.cpu().double() - want).abs() / want.abs().clamp_min(1.0)).max().item() < 1e-5
    assert kernels.gemm_tcgen05_residual(rnd((65, K), 1, torch.bfloat16).to(DEV), w,
                                         torch.zeros((65, N), device=DEV), S) is False


@pytest.mark.parametrize("M,N,K,bias", [(300, 512, 320, True), (257, 400, 1024, False), (2048, 4096, 512, False),
                                        (700, 264, 4096, True)])
def test_gemm_tcgen05_many_rows_add_into_the_residual_stream(M, N, K, bias):
    """The product of many rows is added into the float32 residual by the product's own epilogue: the
    same sums as the separate product followed by the addition, rows and columns beyond the tiles'
    edges included, rows past M untouched."""
    from rocml_b200 import kernels
    x = rnd((M, K), 4, torch.bfloat16).to(DEV)
    w = rnd((N, K), 5, torch.bfloat16, 0.05).to(DEV)
    b = rnd((N,), 6).to(DEV) if bias else None
    resid0 = rnd((M + 3, N), 8)
    resid = resid0.clone().to(DEV)
    assert kernels.gemm_tcgen05_add(x, w, resid, b, M)
    kernels.check_status(DEV)
    want = resid0[:M].double() + x.cpu().double() @ w.cpu().double().t() + (b.cpu().double() if bias else 0.0)
    scale = (x.cpu().double().abs() @ w.cpu().double().abs().t()).clamp_min(1.0)     # as for the plain product
    assert ((resid[:M].cpu().double() - want).abs() / scale).max().item() < 1e-5
    assert torch.equal(resid[M:].cpu(), resid0[M:])
    # and bit for bit what the plain product and a float32 addition give
    delta = torch.empty((M, N), dtype=torch.float32, device=DEV)
    assert kernels.gemm_tcgen05(x, w, delta, b, M)
    assert torch.equal(resid[:M], resid0[:M].to(DEV) + delta)
    assert kernels.gemm_tcgen05_add(x[:200], w, resid, b, 200) is False          # few rows: other kernels


@pytest.mark.parametrize("M,nq,nkv,K,norm,rope,bias,writes", [
    (300, 4, 2, 512, True, True, False, True), (1000, 6, 1, 264, True, True, True, True),
    (513, 2, 2, 1024, False, True, False, True), (257, 4, 2, 256, True, False, False, False)])
@pytest.mark.parametrize("eps", [1e-6, 1e-1])
def test_gemm_tcgen05_qkv_projection_rotates_and_caches(M, nq, nkv, K, norm, rope, bias, writes, eps):
    """A prompt's q | k | v projection whose epilogue does the per-head norm, the rotation and the cache
    write, against the same arithmetic in float64; some tokens are padding and must leave no trace.
    The second eps is as large as the heads' mean squares, so that an eps that is dropped or added in
    the wrong place shows above the bfloat16 tolerance (the 32-bit path never runs this kernel)."""
    from rocml_b200 import kernels
    hd = 128
    g = torch.Generator().manual_seed(M + K)
    N = (nq + 2 * nkv) * hd if writes else nq * hd
    x = (torch.randn((M, K), generator=g) * 0.5).bfloat16()
    w = (torch.randn((N, K), generator=g) * 0.05).bfloat16()
    b = torch.randn((N,), generator=g) * 0.1 if bias else None
    qw = 1 + 0.1 * torch.randn(hd, generator=g) if norm else None
    kw = 1 + 0.1 * torch.randn(hd, generator=g) if norm else None
    # three sequences interleaved token by token: every (slot, page) has a page of its own and every
    # token its own place in it
    pos = torch.arange(M, dtype=torch.int32) // 3 + 40
    slot = torch.arange(M, dtype=torch.int32) % 3
    table = torch.full((3, 12), -1, dtype=torch.int32)
    table[:, :10] = torch.randperm(30, generator=g).reshape(3, 10).to(torch.int32)
    slot[5] = -1
    slot[M - 1] = -1
    n_pages = 31
    kc = torch.zeros((n_pages, max(nkv, 1), 64, hd), dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    inv_freq = (1e4 ** (-torch.arange(0, hd // 2, dtype=torch.float64) * 2 / hd)).float().to(DEV)
    cs = kernels.rope_table(pos.to(DEV), inv_freq, M) if rope else None
    q = torch.zeros((M, nq * hd), dtype=torch.bfloat16, device=DEV)
    assert kernels.gemm_tcgen05_qkv_rope(
        x.to(DEV), w.to(DEV), q, nq, nkv, qw.to(DEV) if norm else None, kw.to(DEV) if norm else None, eps, cs,
        pos.to(DEV), slot.to(DEV), table.to(DEV) if writes else None, kc if writes else None, vc if writes else None,
        b.to(DEV) if bias else None)
    kernels.check_status(DEV)
    proj = x.double() @ w.double().t() + (b.double() if bias else 0)
    heads = proj.reshape(M, -1, hd)

    def finish(h, wn):
        if wn is not None:
            h = h * torch.rsqrt((h * h).mean(-1, keepdim=True) + eps) * wn.double()
        if rope:
            ang = pos.double()[:, None] * inv_freq.cpu().double()[None, :]
            c, sn = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
            lo, hi = h[..., :64], h[..., 64:]
            h = torch.cat([lo * c - hi * sn, lo * sn + hi * c], -1)
        return h
    want_q = finish(heads[:, :nq], qw)
    live = slot >= 0
    got_q = q.cpu().double().reshape(M, nq, hd)
    assert ((got_q[live] - want_q[live]).abs() / want_q[live].abs().clamp_min(1.0)).max() < 2 ** -7
    assert got_q[~live].abs().sum() == 0
    if writes:
        want_k, want_v = finish(heads[:, nq:nq + nkv], kw), heads[:, nq + nkv:]
        seen = 0
        for t in range(M):
            if slot[t] < 0:
                continue
            page, r = int(table[slot[t], pos[t] // 64]), int(pos[t] % 64)
            assert ((kc[page, :, r].cpu().double() - want_k[t]).abs() / want_k[t].abs().clamp_min(1.0)).max() < 2 ** -7
            assert ((vc[page, :, r].cpu().double() - want_v[t]).abs() / want_v[t].abs().clamp_min(1.0)).max() < 2 ** -7
            seen += 1
        assert int((kc.float().abs().sum(-1) > 0).sum()) <= seen * nkv     # nothing written elsewhere


def test_gemm_tcgen05_refuses_unaligned_k():
    from rocml_b200 import kernels
    x = rnd((4, 100), 1, torch.bfloat16).to(DEV)  # K = 100: rows are not a multiple of 16 bytes
    w = rnd((32, 100), 2, torch.bfloat16).to(DEV)
    out = torch.empty((4, 32), dtype=torch.float32, device=DEV)
    assert kernels.gemm_tcgen05(x, w, out) is False


@pytest.mark.parametrize("M,N,K", [(1, 37, 50), (3, 311, 96), (70, 130, 100), (200, 64, 33), (129, 257, 1000), (300, 65, 16),
                                   (2048, 512, 264)])
@pytest.mark.parametrize("xd,wd,od", [(torch.float32, torch.float32, torch.float32),
                                      (torch.bfloat16, torch.bfloat16, torch.bfloat16),
                                      (torch.bfloat16, torch.bfloat16, torch.float32),
                                      (torch.float32, torch.bfloat16, torch.float32)])
def test_gemm_generic(M, N, K, xd, wd, od):
    from rocml_b200 import kernels
    x = rnd((M, K), 1, xd).to(DEV)
    w = rnd((N, K), 2, wd).to(DEV)
    bias = rnd((N,), 3).to(DEV)
    out = torch.full((M, N), float("nan"), dtype=od, device=DEV)
    kernels.gemm_generic(x, w, out, bias)
    want = x.cpu().double() @ w.cpu().double().t() + bias.cpu().double()
    scale = torch.maximum((x.cpu().double().abs() @ w.cpu().double().abs().t()).clamp_min(1.0), want.abs())
    tol = 2 ** -8 if od == torch.bfloat16 else 1e-5
    assert ((out.cpu().double() - want).abs() / scale).max().item() < tol


@pytest.mark.parametrize("M,N,K", [(1, 37, 52), (2, 311, 96), (3, 5, 4), (5, 129, 1000), (8, 4096, 4096), (9, 16, 260),
                                   (16, 1001, 12288), (8, 50, 128)])
def test_gemm_of_few_32_bit_rows_reads_the_weight_once(M, N, K):
    """The 32-bit path's decode product (at most 16 rows, k a multiple of 4): a kernel of its own; a
    row's result does not depend on the rows beside it, and rows of a strided view work."""
    from rocml_b200 import kernels
    wide = rnd((M, K + 8), 1).to(DEV)
    x = wide[:, :K]                                   # a row stride that is not K
    w = rnd((N, K), 2).to(DEV)
    bias = rnd((N,), 3).to(DEV)
    out = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
    kernels.gemm_generic(x, w, out, bias)
    want = x.cpu().double() @ w.cpu().double().t() + bias.cpu().double()
    scale = (x.cpu().double().abs() @ w.cpu().double().abs().t()).clamp_min(1.0)
    assert ((out.cpu().double() - want).abs() / scale).max().item() < 1e-6
    alone = torch.empty((1, N), dtype=torch.float32, device=DEV)
    kernels.gemm_generic(x[M - 1:M].contiguous(), w, alone, bias)
    assert torch.equal(alone[0], out[M - 1])


@pytest.mark.parametrize("M,N,K,S", [(1, 37, 2048, 2), (8, 4096, 4096, 4), (5, 129, 1100, 3), (16, 1001, 12288, 8), (3, 64, 520, 2), (8, 264, 7616, 7)])
def test_gemm_of_few_32_bit_rows_in_parts_of_k(M, N, K, S):
    """The same product with the sum over K in S parts, each a partial result of its own (the bias in the
    first): their sum is the product, every part is written (none stays NaN), and a part is the product
    over its own stretch of k (a multiple of 256 long)."""
    from rocml_b200 import kernels
    x = rnd((M, K), 1).to(DEV)
    w = rnd((N, K), 2).to(DEV)
    bias = rnd((N,), 3).to(DEV)
    out = torch.full((S, M + 1, N), float("nan"), dtype=torch.float32, device=DEV)[:, :M]
    kernels.gemm_generic(x, w, out, bias)
    want = x.cpu().double() @ w.cpu().double().t() + bias.cpu().double()
    scale = (x.cpu().double().abs() @ w.cpu().double().abs().t()).clamp_min(1.0)
    assert not torch.isnan(out).any()
    assert ((out.cpu().double().sum(0) - want).abs() / scale).max().item() < 1e-6
    per = -(-(-(-K // S)) // 256) * 256
    part1 = x.cpu().double()[:, per:2 * per] @ w.cpu().double()[:, per:2 * per].t()
    assert ((out[1].cpu().double() - part1).abs() / scale).max().item() < 1e-6
    # parts that the rounding to tiles leaves empty are zeros; many rows are refused
    few = torch.full((S, M, N), float("nan"), dtype=torch.float32, device=DEV)
    kernels.gemm_generic(x[:, :256].contiguous(), w[:, :256].contiguous(), few, bias)
    assert torch.equal(few[1:], torch.zeros_like(few[1:]))
    part0 = x.cpu().double()[:, :256] @ w.cpu().double()[:, :256].t() + bias.cpu().double()
    assert ((few[0].cpu().double() - part0).abs() / scale).max().item() < 1e-6
    with pytest.raises(kernels.KernelError):
        kernels.gemm_generic(rnd((17, K), 4).to(DEV), w, torch.empty((S, 17, N), device=DEV), bias)


# ---- embedding, norm, activation ---------------------------------------------------------------------

@pytest.mark.parametrize("wd", [torch.float32, torch.bfloat16])
def test_embedding(wd):
    from rocml_b200 import kernels
    table = rnd((333, 72), 1, wd).to(DEV)
    ids = torch.tensor([0, 332, 5, 5, 17], dtype=torch.int32, device=DEV)
    out = torch.empty((5, 72), dtype=torch.float32, device=DEV)
    kernels.embedding(ids, table, out, kernels.status_word(DEV))
    assert torch.equal(out.cpu(), table.cpu().float()[ids.cpu().long()])


def test_embedding_reports_a_bad_id():
    from rocml_b200 import kernels
    from rocml_b200.errors import KernelError
    table = rnd((10, 8), 1).to(DEV)
    ids = torch.tensor([3, 10], dtype=torch.int32, device=DEV)
    out = torch.empty((2, 8), dtype=torch.float32, device=DEV)
    kernels.embedding(ids, table, out, kernels.status_word(DEV))
    with pytest.raises(KernelError):
        kernels.check_status(DEV)
    kernels.check_status(DEV)  # cleared


@pytest.mark.parametrize("H,T", [(72, 7), (1000, 7), (4096, 7), (5120, 7), (4096, 150), (1000, 90), (5120, 70), (8200, 66)])
@pytest.mark.parametrize("od,wd", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                   (torch.bfloat16, torch.float32)])
def test_add_rmsnorm(H, T, od, wd):
    """Few rows (a block's shared memory holds the row) and many rows (the row stays in registers)."""
    from rocml_b200 import kernels
    S, eps = 3, 1e-5
    resid = rnd((T, H), 1, scale=2.0)
    delta = rnd((S, T, H), 2)
    w = (1 + 0.1 * rnd((H,), 3)).to(wd)
    r_dev, d_dev = resid.to(DEV), delta.to(DEV)
    out = torch.empty((T, H), dtype=od, device=DEV)
    kernels.add_rmsnorm(r_dev, d_dev, w.to(DEV), eps, out)
    r = resid.double() + delta.double().sum(0)
    want = r * torch.rsqrt((r * r).mean(-1, keepdim=True) + eps) * w.double()
    assert (r_dev.cpu().double() - r).abs().max() < 1e-5
    tol = 2 ** -7 if od == torch.bfloat16 else 1e-5
    assert ((out.cpu().double() - want).abs() / want.abs().clamp_min(1.0)).max() < tol
    # gathered rows, no write-back, a skipped row
    rows = torch.tensor([4, -1, 0], dtype=torch.int32, device=DEV)
    r2 = resid.to(DEV)
    out2 = torch.zeros((3, H), dtype=od, device=DEV)
    kernels.add_rmsnorm(r2, d_dev, w.to(DEV), eps, out2, rows=rows, write_back=False)
    assert torch.equal(r2.cpu(), resid)
    assert ((out2[[0, 2]].cpu().double() - want[[4, 0]]).abs() / want[[4, 0]].abs().clamp_min(1.0)).max() < tol
    assert out2[1].abs().sum() == 0


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_silu_mul(dt):
    from rocml_b200 import kernels
    T, I = 9, 208
    x = rnd((T, 2 * I), 1, dt, scale=3.0).to(DEV)
    out = torch.empty((T, I), dtype=dt, device=DEV)
    kernels.silu_mul(x, out)
    g, u = x.cpu().double()[:, :I], x.cpu().double()[:, I:]
    want = g / (1 + torch.exp(-g)) * u
    tol = 2 ** -8 if dt == torch.bfloat16 else 1e-6
    assert ((out.cpu().double() - want).abs() / want.abs().clamp_min(1.0)).max() < tol
    parts = torch.stack([x.float() * 0.75, x.float() * 0.25])      # two float32 partial sums
    out2 = torch.empty((T, I), dtype=dt, device=DEV)
    kernels.silu_mul(parts, out2)
    assert ((out2.cpu().double() - want).abs() / want.abs().clamp_min(1.0)).max() < tol
    # gates and ups alternating in blocks of 16 columns
    xc = x.cpu()
    mixed = torch.stack([xc[:, :I].reshape(T, I // 16, 16), xc[:, I:].reshape(T, I // 16, 16)], 2).reshape(T, 2 * I)
    out3 = torch.empty((T, I), dtype=dt, device=DEV)
    kernels.silu_mul(mixed.contiguous().to(DEV), out3, paired=True)
    assert torch.equal(out3, out)


# ---- attention over the paged cache --------------------------------------------------------------------

def paged_case(seed, lens, q_lens, nq, nkv, hd, dtype, spike=None):
    """Sequences with caches of `lens` tokens whose last `q_lens` tokens are this step's queries.
    Pages are handed out in a scrambled order so that a wrong table shows.  `spike` = (seq, far
    key position): that key and the last query of the sequence are scaled so that one far score
    stands out among hundreds."""
    g = torch.Generator().manual_seed(seed)
    B = len(lens)
    n_pages = sum((n + 63) // 64 for n in lens) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    max_pages = max((n + 63) // 64 for n in lens) + 1
    table = torch.full((B + 2, max_pages), -1, dtype=torch.int32)
    slots = list(range(1, B + 1))           # slot 0 stays unused
    kc = torch.full((n_pages, nkv, 64, hd), float("nan"))
    vc = torch.full((n_pages, nkv, 64, hd), float("nan"))
    ks, vs, qs = [], [], []
    for b, n in enumerate(lens):
        k = torch.randn(n, nkv, hd, generator=g)
        v = torch.randn(n, nkv, hd, generator=g)
        q = torch.randn(q_lens[b], nq, hd, generator=g)
        if spike is not None and spike[0] == b:
            k[spike[1]] *= 4.0
            q[-1] = k[spike[1]].repeat_interleave(nq // nkv, dim=0) * 1.5
        k, v, q = k.to(dtype).float(), v.to(dtype).float(), q.to(dtype).float()
        for p in range((n + 63) // 64):
            page = perm.pop()
            table[slots[b], p] = page
            m = min(64, n - p * 64)
            kc[page, :, :m] = k[p * 64:p * 64 + m].transpose(0, 1)
            vc[page, :, :m] = v[p * 64:p * 64 + m].transpose(0, 1)
        ks.append(k); vs.append(v); qs.append(q)
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    meta = dict(table=table, seq_slot=torch.tensor(slots, dtype=torch.int32),
                cu_q=torch.tensor(cu, dtype=torch.int32), kv_len=torch.tensor(lens, dtype=torch.int32))
    return ks, vs, qs, kc.to(dtype), vc.to(dtype), meta


def reference_attention(ks, vs, qs, window, scale):
    import plain_qwen3 as P
    outs = []
    for k, v, q in zip(ks, vs, qs):
        n, ql = k.shape[0], q.shape[0]
        full_q = torch.zeros(n, q.shape[1], q.shape[2], dtype=torch.float64)
        full_q[n - ql:] = q.double()
        o = P.attention(full_q, k.double(), v.double(), window=window, scale=scale)
        outs.append(o[n - ql:])
    return torch.cat(outs, 0)


ATT_CASES = [
    # lens, q_lens, nq, nkv, hd, window
    ([5, 70, 129], [5, 70, 129], 4, 2, 16, None),        # whole prompts
    ([200, 64, 1], [30, 1, 1], 6, 1, 32, None),          # a piece of a prompt, single tokens; 6:1 groups
    ([300, 131], [300, 3], 5, 5, 48, 24),                # a window, no grouping, head size 48
    ([700], [1], 32, 8, 128, None),                      # one far key among hundreds
    ([260, 90], [65, 90], 20, 1, 64, 100),               # a group wider than a block's 16 rows
]


@pytest.mark.parametrize("case", range(len(ATT_CASES)))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_generic(case, dtype):
    from rocml_b200 import kernels
    lens, q_lens, nq, nkv, hd, window = ATT_CASES[case]
    spike = (0, 3) if case == 3 else None
    ks, vs, qs, kc, vc, meta = paged_case(case, lens, q_lens, nq, nkv, hd, dtype, spike)
    scale = 1.0 / math.sqrt(hd)
    want = reference_attention(ks, vs, qs, window, scale)
    q = torch.cat(qs, 0).reshape(-1, nq * hd).to(dtype).to(DEV)
    out = torch.full_like(q, float("nan"))
    d = {k: v.to(DEV) for k, v in meta.items()}
    kernels.attention_generic(q, out, kc.to(DEV), vc.to(DEV), d["table"], d["seq_slot"], d["cu_q"], d["kv_len"],
                              len(lens), max(q_lens), nq, nkv, hd, scale, window or 0)
    tol = 2e-2 if dtype == torch.bfloat16 else 2e-5
    err = (out.cpu().double().reshape(want.shape) - want).abs().max().item()
    assert err < tol, err


PRE_CASES = [
    # lens, q_lens, nq, nkv, hd, window
    ([5, 70, 129, 64], [5, 70, 129, 64], 8, 2, 64, None),      # whole prompts of unequal length
    ([700, 200, 65], [190, 1, 65], 8, 2, 128, None),           # pieces of prompts and a single token
    ([300, 131], [300, 3], 4, 4, 128, 24),                     # a window narrower than a tile
    ([900], [333], 6, 1, 64, 200),                             # a window that spans tiles; 6:1 groups
    ([513], [513], 2, 1, 256, None),
]


@pytest.mark.parametrize("case", range(len(PRE_CASES)))
def test_attention_prefill_tensor_cores(case):
    from rocml_b200 import kernels
    lens, q_lens, nq, nkv, hd, window = PRE_CASES[case]
    dtype = torch.bfloat16
    spike = (0, 2) if case == 1 else None         # a far key that outweighs hundreds of near ones
    ks, vs, qs, kc, vc, meta = paged_case(20 + case, lens, q_lens, nq, nkv, hd, dtype, spike)
    scale = 1.0 / math.sqrt(hd)
    want = reference_attention(ks, vs, qs, window, scale)
    q = torch.cat(qs, 0).reshape(-1, nq * hd).to(dtype).to(DEV)
    out = torch.full_like(q, float("nan"))
    d = {k: v.to(DEV) for k, v in meta.items()}
    kc, vc = kc.to(DEV), vc.to(DEV)
    kc[kc != kc] = 1e30      # what lies beyond a sequence's end in its last page must not matter
    vc[vc != vc] = 1e30
    assert kernels.attention_prefill(q, out, kc, vc, d["table"], d["seq_slot"], d["cu_q"], d["kv_len"], len(lens),
                                     max(q_lens), nq, nkv, hd, scale, window or 0)
    err = (out.cpu().double().reshape(want.shape) - want).abs().max().item()
    assert err < 2e-2, err


TC5_CASES = [
    PRE_CASES[1],
    PRE_CASES[2],
    ([1000, 333, 129, 64], [1000, 77, 129, 1], 4, 2, 128, None),   # several tiles of 256 queries; pieces that start anywhere
    ([900], [600], 2, 1, 128, 200),                                # a window that spans tiles of 128 keys
    ([520, 257], [520, 130], 3, 3, 128, 130),                      # a window about as wide as a tile; a last tile of one page
    ([448, 449, 385], [448, 449, 2], 2, 2, 128, None),             # lengths around the edges of pages and tiles
    PRE_CASES[0],                                                  # head size 64
    PRE_CASES[3],                                                  # head size 64, a window, 6:1 groups
    PRE_CASES[4],                                                  # head size 256
    ([700, 130], [450, 130], 4, 2, 256, 150),                      # head size 256: a piece of a prompt, a window
]


@pytest.mark.parametrize("case", range(len(TC5_CASES)))
def test_attention_prefill_tcgen05(case):
    """The tensor-memory kernel (head size 128): pieces of prompts, windows, lengths around the tiles' edges."""
    from rocml_b200 import kernels
    lens, q_lens, nq, nkv, hd, window = TC5_CASES[case]
    dtype = torch.bfloat16
    spike = (0, 2) if case == 0 else None
    ks, vs, qs, kc, vc, meta = paged_case(20 + case, lens, q_lens, nq, nkv, hd, dtype, spike)
    scale = 1.0 / math.sqrt(hd)
    want = reference_attention(ks, vs, qs, window, scale)
    q = torch.cat(qs, 0).reshape(-1, nq * hd).to(dtype).to(DEV)
    out = torch.full_like(q, float("nan"))
    d = {k: v.to(DEV) for k, v in meta.items()}
    kc, vc = kc.to(DEV), vc.to(DEV)      # beyond a sequence's end the pages hold NaN: it must not matter
    assert kernels.attention_prefill_tc5(q, q.shape[0], out, kc, vc, d["table"], d["seq_slot"], d["cu_q"], d["kv_len"],
                                         len(lens), max(q_lens), nq, nkv, hd, scale, window or 0)
    kernels.check_status(DEV)
    err = (out.cpu().double().reshape(want.shape) - want).abs().max().item()
    assert err < 2e-2, err


@pytest.mark.parametrize("nq,nkv,q_len,kv_len,spread,window", [
    (32, 8, 4096, 4096, 1.0, 0), (4, 2, 4096, 4096, 4.0, 0), (32, 8, 104, 4200, 1.0, 0), (8, 8, 1500, 1500, 6.0, 0),
    (32, 8, 3000, 3000, 3.0, 700)])
def test_attention_prefill_tcgen05_with_every_multiprocessor_busy(nq, nkv, q_len, kv_len, spread, window):
    """Thousands of blocks, two a multiprocessor, and scores spread widely enough that the running maxima move
    often: what depends on the order in which a block's roles get to run shows here.  Against the mma.sync
    kernel, which shares no code with it."""
    from rocml_b200 import kernels
    hd = 128
    g = torch.Generator().manual_seed(nq * 1000 + q_len)
    n_pages = (kv_len + 63) // 64
    q = (torch.randn(q_len, nq * hd, generator=g) * spread).bfloat16().to(DEV)
    kc = torch.randn(n_pages, nkv, 64, hd, generator=g).bfloat16().to(DEV)
    vc = torch.randn(n_pages, nkv, 64, hd, generator=g).bfloat16().to(DEV)
    table = torch.arange(n_pages, dtype=torch.int32, device=DEV).reshape(1, n_pages)
    seq_slot = torch.zeros(1, dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, q_len], dtype=torch.int32, device=DEV)
    kv = torch.tensor([kv_len], dtype=torch.int32, device=DEV)
    got, want = torch.full_like(q, float("nan")), torch.full_like(q, float("nan"))
    scale = 1.0 / math.sqrt(hd)
    first = None
    for _ in range(8):       # the order in which roles run differs from launch to launch
        assert kernels.attention_prefill_tc5(q, q_len, got, kc, vc, table, seq_slot, cu, kv, 1, q_len, nq, nkv, hd, scale, window,
                                             max_kv_len=kv_len)
        assert kernels.attention_prefill(q, want, kc, vc, table, seq_slot, cu, kv, 1, q_len, nq, nkv, hd, scale, window)
        kernels.check_status(DEV)
        err = (got.float() - want.float()).abs().max().item()
        assert err < 3e-2, err
        first = got.clone() if first is None else first
        assert torch.equal(got, first)        # the same work gives the same bits, whatever order the blocks and warps ran in
        got.fill_(float("nan"))


DEC_CASES = [
    # lens, nq, nkv, hd, window
    ([700, 1, 129, 64, 128], 32, 8, 128, None),
    ([300, 131, 65], 8, 2, 64, None),
    ([513, 40], 6, 3, 128, 70),
    ([1000], 2, 2, 256, None),
    ([257, 100, 31], 12, 2, 64, 33),
]


@pytest.mark.parametrize("case", range(len(DEC_CASES)))
@pytest.mark.parametrize("fast", [True, False, 3, 100, "shared", "shared-2", "shared-1"])
def test_attention_decode_split_kv(case, fast):
    """One query per sequence, keys in chunks of 128, merged: the bfloat16 kernel and the plain kernel."""
    from rocml_b200 import kernels
    lens, nq, nkv, hd, window = DEC_CASES[case]
    spike = (0, 5) if case == 0 else None
    dtype = torch.bfloat16
    ks, vs, qs, kc, vc, meta = paged_case(10 + case, lens, [1] * len(lens), nq, nkv, hd, dtype, spike)
    scale = 1.0 / math.sqrt(hd)
    want = reference_attention(ks, vs, qs, window, scale)
    B = len(lens)
    q = torch.cat(qs, 0).reshape(-1, nq * hd).to(dtype).to(DEV)
    out = torch.full_like(q, float("nan"))
    d = {k: v.to(DEV) for k, v in meta.items()}
    ppb = 1 if fast in (True, False) else fast        # pages per block of the bfloat16 kernel
    if isinstance(fast, str):
        # a fixed number of blocks a head group, which share the pages of all sequences equally: more
        # blocks than sequences, or fewer (a block then ends one sequence and begins the next)
        ppb, n_chunks = 0, (len(lens) + 6 if fast == "shared" else int(fast[-1]))
    else:
        n_chunks = ((max(lens) + 63) // 64 + ppb - 1) // ppb + 1     # one more than needed, as a padded graph would have
    acc = torch.full((B, nq, n_chunks, hd), float("nan"), dtype=torch.float32, device=DEV)
    ml = torch.full((B, nq, n_chunks, 2), float("nan"), dtype=torch.float32, device=DEV)
    if n_chunks == 1:
        acc = ml = None
    pos = (d["kv_len"] - 1).to(torch.int32)
    if fast:
        assert kernels.attention_decode(q, out, kc.to(DEV), vc.to(DEV), d["table"], d["seq_slot"], d["cu_q"],
                                        d["kv_len"], B, nq, nkv, hd, scale, window or 0, n_chunks, acc, ml, ppb)
        assert int(kernels.decode_counters(DEV).abs().sum()) == 0      # the work space is left zeroed
    else:
        kernels.attention_generic(q, out, kc.to(DEV), vc.to(DEV), d["table"], d["seq_slot"], d["cu_q"], d["kv_len"],
                                  B, 1, nq, nkv, hd, scale, window or 0, 64, n_chunks, acc, ml)
        kernels.attention_merge(acc, ml, out, pos, d["seq_slot"], B, nq, hd, 64, n_chunks, window or 0)
    err = (out.cpu().double().reshape(want.shape) - want).abs().max().item()
    assert err < 2e-2, err


@pytest.mark.parametrize("lens,nq,nkv,window,S,norm,rope,grid", [
    ([700, 1, 129, 64, 128], 32, 8, None, 7, True, True, (1, 1)),      # one page per block: clusters of up to 12
    ([300, 131, 65], 8, 2, None, 1, True, True, (2, 3)),               # clusters of 2
    ([513, 40], 6, 3, 70, 3, False, True, (1, 1)),                    # a window, no per-head norm
    ([1100], 32, 2, None, 2, True, False, (1, 1)),                     # 16 query heads per group: a full tile; 18 chunks: merged through global memory
    ([900, 70, 300, 5], 8, 2, None, 4, True, True, (0, 9)),            # nine blocks a group share the pages
    ([900, 70, 300, 5, 64, 65, 200], 8, 2, None, 4, True, True, (0, 3)),  # fewer blocks than sequences
    ([130, 70, 300], 8, 2, 100, 2, True, True, (0, 2)),                # the same with a window
])
@pytest.mark.parametrize("eps", [1e-6, 1e-1])
def test_attention_decode_takes_the_projections_itself(lens, nq, nkv, window, S, norm, rope, grid, eps):
    """Head size 128: the decode kernel is given the projection's partial sums and does the
    per-head norm, the rotation and the cache write of the new token itself.  Same output and same
    cache as the two kernels one after the other, and the right output by float64.  The second eps is
    of the size of the heads' mean squares, so that a dropped or misplaced eps shows."""
    from rocml_b200 import kernels
    hd, B = 128, len(lens)
    ks, vs, qs, kc, vc, meta = paged_case(31, lens, [1] * B, nq, nkv, hd, torch.bfloat16)
    d = {k: v.to(DEV) for k, v in meta.items()}
    gen = torch.Generator().manual_seed(5)
    width = (nq + 2 * nkv) * hd
    proj = (torch.randn((S, B, width), generator=gen) * (1.0 / S)).to(DEV)
    qw = (1 + 0.1 * torch.randn(hd, generator=gen)).to(DEV) if norm else None
    kw = (1 + 0.1 * torch.randn(hd, generator=gen)).to(DEV) if norm else None
    pos = (d["kv_len"] - 1).to(torch.int32)
    slot_of_token = d["seq_slot"]
    inv_freq = (1e6 ** (-torch.arange(0, hd // 2, dtype=torch.float64) * 2 / hd)).float().to(DEV) if rope else None
    cs = kernels.rope_table(pos, inv_freq, B) if rope else None
    scale = 1.0 / math.sqrt(hd)
    ppb, shared_blocks = grid
    n_chunks = shared_blocks if ppb == 0 else ((max(lens) + 63) // 64 + ppb - 1) // ppb
    outs, caches = [], []
    for fused in (False, True):
        k2, v2 = kc.clone().to(DEV), vc.clone().to(DEV)
        out = torch.full((B, nq * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        acc = torch.empty((B, nq, n_chunks, hd), dtype=torch.float32, device=DEV)
        ml = torch.empty((B, nq, n_chunks, 2), dtype=torch.float32, device=DEV)
        if fused:
            assert kernels.attention_decode_fused(proj, out, k2, v2, d["table"], d["seq_slot"], d["cu_q"], d["kv_len"],
                                                  B, nq, nkv, hd, qw, kw, eps, cs, True, scale, window or 0,
                                                  n_chunks, acc, ml, ppb)
        else:
            q = torch.empty((B, nq * hd), dtype=torch.bfloat16, device=DEV)
            kernels.qk_norm_rope_cache(proj, q, B, nq, nkv, hd, qw, kw, eps, inv_freq, hd if rope else 0, pos,
                                       slot_of_token, d["table"], k2, v2, write_kv=True, cos_sin=cs)
            assert kernels.attention_decode(q, out, k2, v2, d["table"], d["seq_slot"], d["cu_q"], d["kv_len"], B, nq,
                                            nkv, hd, scale, window or 0, n_chunks, acc, ml, ppb)
        assert int(kernels.decode_counters(DEV).abs().sum()) == 0
        outs.append(out.float().cpu())
        caches.append((torch.nan_to_num(k2.float()).cpu(), torch.nan_to_num(v2.float()).cpu()))
    assert torch.isfinite(outs[1]).all()
    assert torch.equal(caches[0][0], caches[1][0]) and torch.equal(caches[0][1], caches[1][1])
    assert (outs[0] - outs[1]).abs().max().item() < 1e-2
    # float64: the new token's key and value from the summed projections, the other keys from the cache
    import plain_qwen3 as P
    summed = proj.double().sum(0).cpu().reshape(B, nq + 2 * nkv, hd)
    qh, kh, vh = summed[:, :nq], summed[:, nq:nq + nkv], summed[:, nq + nkv:]
    if norm:
        qh, kh = P.rmsnorm(qh, qw.double().cpu(), eps), P.rmsnorm(kh, kw.double().cpu(), eps)
    if rope:
        qh = torch.stack([P.rope_neox(qh[b:b + 1], [lens[b] - 1], 1e6)[0] for b in range(B)])
        kh = torch.stack([P.rope_neox(kh[b:b + 1], [lens[b] - 1], 1e6)[0] for b in range(B)])
    for b, n in enumerate(lens):
        keys = torch.cat([ks[b][:n - 1].double(), kh[b:b + 1].bfloat16().double()])       # [n, nkv, hd]
        vals = torch.cat([vs[b][:n - 1].double(), vh[b:b + 1].bfloat16().double()])
        lo = max(0, n - window) if window else 0
        for h in range(nq):
            kv = h // (nq // nkv)
            sc = (keys[lo:, kv] @ qh[b, h].bfloat16().double()) * scale
            want = torch.softmax(sc, 0) @ vals[lo:, kv]
            assert (outs[1][b, h * hd:(h + 1) * hd].double() - want).abs().max().item() < 2e-2, (b, h)


def test_attention_decode_leaves_wide_groups_to_the_two_kernels():
    """More than 16 query heads a key/value head: several blocks would read the new token's page while
    one of them writes it, so the kernel that takes the projections declines (the caller then writes
    the cache with the kernel of its own); when it only reads a cache that is written already it runs."""
    from rocml_b200 import kernels
    hd, nq, nkv, lens = 128, 40, 2, [200, 70]
    B = len(lens)
    ks, vs, qs, kc, vc, meta = paged_case(3, lens, [1] * B, nq, nkv, hd, torch.bfloat16)
    d = {k: v.to(DEV) for k, v in meta.items()}
    n_chunks = (max(lens) + 63) // 64
    out = torch.zeros((B, nq * hd), dtype=torch.bfloat16, device=DEV)
    acc = torch.empty((B, nq, n_chunks, hd), dtype=torch.float32, device=DEV)
    ml = torch.empty((B, nq, n_chunks, 2), dtype=torch.float32, device=DEV)
    k2, v2 = kc.clone().to(DEV), vc.clone().to(DEV)
    before = k2.clone()
    for writes, expect in ((True, False), (False, True)):
        proj = torch.randn((2, B, (nq + (2 * nkv if writes else 0)) * hd), device=DEV)
        got = kernels.attention_decode_fused(proj, out, k2, v2, d["table"], d["seq_slot"], d["cu_q"], d["kv_len"],
                                             B, nq, nkv, hd, None, None, 1e-6, None, writes, 0.1, 0, n_chunks, acc, ml, 1)
        assert got is expect
    assert torch.equal(torch.nan_to_num(k2.float()), torch.nan_to_num(before.float()))
    kernels.check_status(DEV)


def test_attention_decode_refuses_other_head_sizes():
    from rocml_b200 import kernels
    ks, vs, qs, kc, vc, meta = paged_case(1, [10], [1], 2, 1, 48, torch.bfloat16)
    q = torch.cat(qs, 0).reshape(-1, 96).bfloat16().to(DEV)
    d = {k: v.to(DEV) for k, v in meta.items()}
    assert kernels.attention_decode(q, torch.empty_like(q), kc.to(DEV), vc.to(DEV), d["table"], d["seq_slot"],
                                    d["cu_q"], d["kv_len"], 1, 2, 1, 48, 0.1, 0, 1, None, None) is False


# ---- q/k norm + rotary + cache write ---------------------------------------------------------------------

@pytest.mark.parametrize("dtype,wd", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("nq,nkv,hd,rot", [(4, 2, 16, 16), (6, 1, 32, 32), (5, 5, 48, 24), (8, 2, 128, 128)])
def test_qk_norm_rope_cache(dtype, wd, nq, nkv, hd, rot):
    import plain_qwen3 as P
    from rocml_b200 import kernels
    T, eps, theta = 9, 1e-5, 1e4
    positions = torch.tensor([0, 1, 2, 63, 64, 65, 130, 7, 8], dtype=torch.int32)
    slots = torch.tensor([1, 1, 1, 1, 1, 1, 1, 2, -1], dtype=torch.int32)   # the last token is padding
    table = torch.full((3, 4), -1, dtype=torch.int32)
    table[1, :3] = torch.tensor([5, 0, 3])
    table[2, :1] = torch.tensor([2])
    width = (nq + 2 * nkv) * hd
    x = rnd((T, width), 1, dtype)
    qw, kw = (1 + 0.1 * rnd((hd,), 2)).to(wd), (1 + 0.1 * rnd((hd,), 3)).to(wd)
    inv = torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot).float()
    kc = torch.zeros((6, nkv, 64, hd), dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    xd = x.to(DEV).clone()
    kernels.qk_norm_rope_cache(xd, xd, T, nq, nkv, hd, qw.to(DEV), kw.to(DEV), eps, inv.to(DEV), rot, positions.to(DEV),
                               slots.to(DEV), table.to(DEV), kc, vc)
    xf = x.double()
    q = P.rmsnorm(xf[:, :nq * hd].reshape(T, nq, hd), qw.double(), eps)
    k = P.rmsnorm(xf[:, nq * hd:(nq + nkv) * hd].reshape(T, nkv, hd), kw.double(), eps)
    v = xf[:, (nq + nkv) * hd:].reshape(T, nkv, hd)

    def rope(t):
        r = P.rope_neox(t[..., :rot], positions.tolist(), theta)
        return torch.cat([r, t[..., rot:]], -1)
    q, k = rope(q), rope(k)
    tol = 2e-2 if dtype == torch.bfloat16 else 2e-5
    got_q = xd.cpu().double()[:, :nq * hd].reshape(T, nq, hd)
    assert (got_q[:8] - q[:8]).abs().max() < tol
    assert torch.equal(xd.cpu()[8], x[8])                       # the padded token is untouched
    for t in range(8):
        page = int(table[slots[t], positions[t] // 64])
        off = int(positions[t] % 64)
        assert (kc[page, :, off].cpu().double() - k[t]).abs().max() < tol
        assert (vc[page, :, off].cpu().double() - v[t]).abs().max() < tol * 1e-3 + 1e-7
    assert kc.abs().sum(dim=(1, 3)).count_nonzero() == 8         # nothing else was written
    # the same from three float32 partial sums, q into a buffer of its own
    parts = torch.stack([x.float() * 0.5, x.float() * 0.25, x.float() * 0.25]).to(DEV)
    q2 = torch.zeros((T, nq * hd), dtype=dtype, device=DEV)
    kc2, vc2 = torch.zeros_like(kc), torch.zeros_like(vc)
    kernels.qk_norm_rope_cache(parts, q2, T, nq, nkv, hd, qw.to(DEV), kw.to(DEV), eps, inv.to(DEV), rot,
                               positions.to(DEV), slots.to(DEV), table.to(DEV), kc2, vc2)
    assert (q2[:8].cpu().double().reshape(8, nq, hd) - q[:8]).abs().max() < tol
    assert (kc2.cpu().double() - kc.cpu().double()).abs().max() < tol and torch.equal(vc2, vc)


# ---- a bounded wait that runs out ------------------------------------------------------------------------

def test_a_wait_that_runs_out_is_reported_and_the_device_stays_usable():
    """Every barrier wait in the tensor-core kernels has a limit.  Here one runs out: a one-block
    product (8 x 128 x 128) is launched with a limit of 100,000 cycles (tens of microseconds) and
    with its first K block never requested, so the warp that waits for that block gives up.  The
    kernel must record the failure in the status word, let the block unwind (the producer waits for
    the copies it did request, tensor memory is freed) and return; the host raises KernelError and
    clears the word; and the same launch without the switch then gives the right product, which
    shows that the device was left clean.  Nothing traps and nothing spins without limit."""
    from rocml_b200 import kernels
    from rocml_b200.errors import KernelError
    M, N, K = 8, 128, 128
    x = rnd((M, K), 1, torch.bfloat16).to(DEV)
    w = rnd((N, K), 2, torch.bfloat16).to(DEV)
    want = x.cpu().double() @ w.cpu().double().t()
    kernels.check_status(DEV)                       # clean before
    out = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
    kernels.set_wait_limit(100_000, withhold_first_stage=True)
    try:
        t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        assert kernels.gemm_tcgen05(x, w, out)
        t1.record()
        torch.cuda.synchronize()
    finally:
        kernels.set_wait_limit(0, False)
    assert t0.elapsed_time(t1) < 50.0               # milliseconds: it gave up at its limit, not at two seconds
    assert torch.isnan(out).all()                   # an abandoned product writes nothing
    with pytest.raises(KernelError, match="bounded wait"):
        kernels.check_status(DEV)
    kernels.check_status(DEV)                       # reading it cleared it
    for _ in range(2):                              # the same launch, as often as one likes
        out = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
        assert kernels.gemm_tcgen05(x, w, out)
        kernels.check_status(DEV)
        assert (out.cpu().double() - want).abs().max().item() < 1e-3


@pytest.mark.parametrize("seed", range(40))
def test_gemm_tcgen05_random_shapes(seed):
    """Shapes drawn at random (any M, any N, K a multiple of 8 as the kernel asks): whole results in both
    output types and partial sums over K, against float64.  Every kernel of the family is reached: few
    tokens (weights on the 128-row side), many (one CTA, CTA pairs), tails in every dimension."""
    import random
    from rocml_b200 import kernels
    rng = random.Random(seed)
    M = rng.choice([rng.randint(1, 16), rng.randint(17, 128), rng.randint(129, 700), rng.randint(700, 2500)])
    N = rng.choice([rng.randint(1, 64), rng.randint(65, 600), rng.randint(600, 3000)])
    K = 8 * rng.choice([rng.randint(1, 8), rng.randint(9, 64), rng.randint(65, 600)])
    x = rnd((M, K), seed, torch.bfloat16).to(DEV)
    w = rnd((N, K), seed + 1, torch.bfloat16).to(DEV)
    bias = rnd((N,), seed + 2).to(DEV) if rng.random() < 0.5 else None
    want = x.cpu().double() @ w.cpu().double().t() + (bias.cpu().double() if bias is not None else 0)
    scale = torch.maximum((x.cpu().double().abs() @ w.cpu().double().abs().t()).clamp_min(1.0), want.abs())
    for out_dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2 ** -8)):
        out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
        assert kernels.gemm_tcgen05(x, w, out, bias)
        assert ((out.cpu().double() - want).abs() / scale).max().item() < tol, (M, N, K, out_dtype)
    S = rng.choice([2, 3, 4, 8])
    if K // 64 >= S:
        out = torch.full((S, M, N), float("nan"), dtype=torch.float32, device=DEV)
        assert kernels.gemm_tcgen05(x, w, out, bias)
        assert ((out.cpu().double().sum(0) - want).abs() / scale).max().item() < 1e-5, (M, N, K, S)
    kernels.check_status(DEV)
