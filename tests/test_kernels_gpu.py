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


def test_gemm_tcgen05_refuses_unaligned_k():
    from rocml_b200 import kernels
    x = rnd((4, 100), 1, torch.bfloat16).to(DEV)  # K = 100: rows are not a multiple of 16 bytes
    w = rnd((32, 100), 2, torch.bfloat16).to(DEV)
    out = torch.empty((4, 32), dtype=torch.float32, device=DEV)
    assert kernels.gemm_tcgen05(x, w, out) is False


@pytest.mark.parametrize("M,N,K", [(1, 37, 50), (3, 311, 96), (70, 130, 100), (200, 64, 33)])
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
    scale = (x.cpu().double().abs() @ w.cpu().double().abs().t()).clamp_min(1.0)
    tol = 2 ** -8 if od == torch.bfloat16 else 1e-5
    assert ((out.cpu().double() - want).abs() / scale).max().item() < tol


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


@pytest.mark.parametrize("H", [72, 1000, 4096, 5120])
@pytest.mark.parametrize("od,wd", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                   (torch.bfloat16, torch.float32)])
def test_add_rmsnorm(H, od, wd):
    from rocml_b200 import kernels
    T, S, eps = 7, 3, 1e-5
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
