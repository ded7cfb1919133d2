// Plain tiled matrix product on the CUDA cores: out[M, N] = x[M, K] . W[N, K]^T (+ bias[N], 32-bit).
//
// 32-bit FMA accumulation, no tensor cores and no reduced-precision mode, for every element
// type.  It is the matrix product of the true 32-bit path, the fallback for sizes the
// tcgen05 kernel refuses, and the reference the tcgen05 kernel is tested against.  The sum
// over k runs in ascending order for every output element whatever M is, so a row's result
// does not depend on what else is in the batch.  It stands where the reference has
// gemv_f16 / gemm_xwt_f16 (rocml-kernels/kernels/gemv_f16.hip:8-36, gemm_f16.hip:10-41).
#include "common.cuh"
#include "api.h"

using namespace rb;

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename XT, typename WT, typename OT>
__global__ void __launch_bounds__(256)
gemm_tn_kernel(const XT* __restrict__ x, const WT* __restrict__ w, const float* __restrict__ bias,
               OT* __restrict__ out, int M, int N, int K, long long ldx, long long ldo) {
    pdl_trigger();
    pdl_wait();
    __shared__ float xs[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int ty = tid / 16, tx = tid % 16;
    const int lr = tid / 4, lc = (tid % 4) * 4;  // this thread loads row lr, k columns lc..lc+3
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = k0 + lc + j;
            const int m = m0 + lr, n = n0 + lr;
            xs[lc + j][lr] = (m < M && k < K) ? to_f32(x[(size_t)m * ldx + k]) : 0.f;
            ws[lc + j][lr] = (n < N && k < K) ? to_f32(w[(size_t)n * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = xs[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[n];
            out[(size_t)m * ldo + n] = from_f32<OT>(v);
        }
    }
}

template <typename XT, typename WT, typename OT>
int launch(const void* x, const void* w, const void* bias, void* out, int M, int N, int K, long long ldx,
           long long ldo, cudaStream_t s) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return RB_ERR_BAD_SIZE;
    RB_LAUNCH((gemm_tn_kernel<XT, WT, OT>), dim3(grid), dim3(256), 0, s, (const XT*)x, (const WT*)w, (const float*)bias, (OT*)out, M,
                                                    N, K, ldx, ldo);
    RB_LAUNCH_CHECK();
    return RB_OK;
}
}  // namespace

extern "C" int rb_gemm_generic(const void* x, int x_dtype, const void* w, int w_dtype, const void* bias,
                               void* out, int out_dtype, int M, int N, int K, long long ldx, long long ldo,
                               void* stream) {
    if (M <= 0 || N <= 0) return RB_OK;
    if (K <= 0) return RB_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    typedef __nv_bfloat16 bf;
#define RB_G(XT, WT, OT) return launch<XT, WT, OT>(x, w, bias, out, M, N, K, ldx, ldo, s)
    if (x_dtype == RB_F32 && w_dtype == RB_F32 && out_dtype == RB_F32) RB_G(float, float, float);
    if (x_dtype == RB_F32 && w_dtype == RB_BF16 && out_dtype == RB_F32) RB_G(float, bf, float);
    if (x_dtype == RB_BF16 && w_dtype == RB_BF16 && out_dtype == RB_BF16) RB_G(bf, bf, bf);
    if (x_dtype == RB_BF16 && w_dtype == RB_BF16 && out_dtype == RB_F32) RB_G(bf, bf, float);
    if (x_dtype == RB_BF16 && w_dtype == RB_F32 && out_dtype == RB_BF16) RB_G(bf, float, bf);
    if (x_dtype == RB_BF16 && w_dtype == RB_F32 && out_dtype == RB_F32) RB_G(bf, float, float);
#undef RB_G
    return RB_ERR_BAD_DTYPE;
}
