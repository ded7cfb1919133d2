// Plain tiled matrix product on the CUDA cores: out[M, N] = x[M, K] . W[N, K]^T (+ bias[N], 32-bit).
//
// 32-bit FMA accumulation, no tensor cores and no reduced-precision mode, for every element
// type.  It is the matrix product of the true 32-bit path, the fallback for sizes the
// tcgen05 kernel refuses, and the reference the tcgen05 kernel is tested against.  In the tiled
// kernel the sum over k runs in ascending order for every output element whatever M is.  It stands
// where the reference has gemv_f16 / gemm_xwt_f16 (rocml-kernels/kernels/gemv_f16.hip:8-36,
// gemm_f16.hip:10-41).
//
// Few rows of 32-bit operands (a decode step of the 32-bit path) take a second kernel that is bound
// by reading the weight once: a warp owns two weight rows and streams them with 16-byte loads, every
// lane multiplying its slice of k with the same slice of all the step's rows (which a block brings
// into shared memory tile by tile), and the lanes' sums meet in a shuffle tree.  How k is dealt out over the lanes depends on
// nothing but k, so a row's result does not depend on what else is in the batch here either.
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

// ---- many rows: 128 x 128 tiles, 8 x 8 outputs a thread ------------------------------------------------
// The same sum in the same order (k ascending for every output element) on larger tiles: a thread owns
// two groups of four rows and two groups of four columns (64 apart, so that a warp's 16-byte reads of
// shared memory fall on consecutive banks), a tile of k is 16 deep, and the next tile's global loads are
// in flight while this one is multiplied.  2.5 times the small tiles' rate on a prompt of 2,048 tokens.
constexpr int LBM = 128, LBN = 128, LBK = 16, LLD = LBM + 4;

template <typename XT, typename WT, typename OT>
__global__ void __launch_bounds__(256, 2)
gemm_tn_large_kernel(const XT* __restrict__ x, const WT* __restrict__ w, const float* __restrict__ bias,
                     OT* __restrict__ out, int M, int N, int K, long long ldx, long long ldo) {
    pdl_trigger();
    pdl_wait();
    __shared__ __align__(16) float xs[2][LBK][LLD];
    __shared__ __align__(16) float ws[2][LBK][LLD];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * LBM, n0 = blockIdx.x * LBN;
    const int ty = tid / 16, tx = tid % 16;
    // loads: thread t brings k columns lc .. lc + 3 of rows lr and lr + 64 of both operands
    const int lr = tid / 4, lc = (tid % 4) * 4;
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
    float xr[2][4], wr[2][4];
    // 32-bit operands whose rows start on 16 bytes are read four k at a time
    const bool x4 = sizeof(XT) == 4 && (ldx & 3) == 0 && ((uintptr_t)x & 15) == 0;
    const bool w4 = sizeof(WT) == 4 && (K & 3) == 0 && ((uintptr_t)w & 15) == 0;
    auto fetch = [&](int k0) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int m = m0 + lr + h * 64, n = n0 + lr + h * 64;
            const int k = k0 + lc;
            if (x4 && m < M && k + 3 < K) {
                const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + (size_t)m * ldx + k);
                xr[h][0] = v.x; xr[h][1] = v.y; xr[h][2] = v.z; xr[h][3] = v.w;
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) xr[h][j] = (m < M && k + j < K) ? to_f32(x[(size_t)m * ldx + k + j]) : 0.f;
            }
            if (w4 && n < N && k + 3 < K) {
                const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w) + (size_t)n * K + k);
                wr[h][0] = v.x; wr[h][1] = v.y; wr[h][2] = v.z; wr[h][3] = v.w;
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) wr[h][j] = (n < N && k + j < K) ? to_f32(w[(size_t)n * K + k + j]) : 0.f;
            }
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                xs[buf][lc + j][lr + h * 64] = xr[h][j];
                ws[buf][lc + j][lr + h * 64] = wr[h][j];
            }
    };
    fetch(0);
    stash(0);
    __syncthreads();
    int buf = 0;
    for (int k0 = 0; k0 < K; k0 += LBK, buf ^= 1) {
        if (k0 + LBK < K) fetch(k0 + LBK);
#pragma unroll
        for (int kk = 0; kk < LBK; ++kk) {
            float a[8], b[8];
            const float4 a0 = *reinterpret_cast<const float4*>(&xs[buf][kk][ty * 4]);
            const float4 a1 = *reinterpret_cast<const float4*>(&xs[buf][kk][64 + ty * 4]);
            const float4 b0 = *reinterpret_cast<const float4*>(&ws[buf][kk][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4*>(&ws[buf][kk][64 + tx * 4]);
            a[0] = a0.x; a[1] = a0.y; a[2] = a0.z; a[3] = a0.w; a[4] = a1.x; a[5] = a1.y; a[6] = a1.z; a[7] = a1.w;
            b[0] = b0.x; b[1] = b0.y; b[2] = b0.z; b[3] = b0.w; b[4] = b1.x; b[5] = b1.y; b[6] = b1.z; b[7] = b1.w;
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (k0 + LBK < K) stash(buf ^ 1);
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + i - 4);
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int n = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + j - 4);
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[n];
            out[(size_t)m * ldo + n] = from_f32<OT>(v);
        }
    }
}

// ---- few rows, 32-bit: one pass over the weight ----------------------------------------------------
constexpr int ROWS_PER_BLOCK = 16;   // weight rows a block: 4 warps of 4 rows (up to 8 step rows) or 8 warps of 2

__device__ __forceinline__ float4 ld_stream(const float* p) {      // read once: do not keep it in the L1
    float4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}

// A block owns 16 weight rows.  k is walked in tiles of KT: the step's rows of a tile are brought
// into shared memory once for the whole block (two buffers, so that the next tile's copy and the next
// tile's weight loads are in flight while this tile is multiplied), and every lane takes the 16-byte
// groups lane, lane + 32, ... of the tile.  A 16-byte group of a step row read from shared memory
// feeds 4 * ROWS_NW multiply-adds: with 4 weight rows a warp the shared-memory reads no longer bound
// the kernel (with 2 they did, at about half the memory's bandwidth).
template <int MT>
__global__ void __launch_bounds__(MT <= 8 ? 128 : 256)
gemm_rows_f32_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                     float* __restrict__ out, int M, int N, int K, long long ldx, long long ldo, int k_per_split,
                     long long split_stride) {
    constexpr int ROWS_NW = MT <= 8 ? 4 : 2;     // weight rows a warp
    constexpr int ROWS_WARPS = ROWS_PER_BLOCK / ROWS_NW;
    constexpr int KT = 256;                      // floats of k a tile
    constexpr int U = KT / 128;                  // 16-byte groups a lane takes of a tile, per row
    __shared__ __align__(16) float xs[2][MT][KT];
    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = (blockIdx.x * ROWS_WARPS + warp) * ROWS_NW;
    // blockIdx.y: this block's part of k (a multiple of KT long); its sums go to a partial result of their own,
    // which the consumer adds in order (a narrow weight alone has too few rows to keep the memory busy)
    const int k_lo = blockIdx.y * k_per_split;
    const int k_end = min(K, k_lo + k_per_split);
    out += (size_t)blockIdx.y * split_stride;
    const float* wr[ROWS_NW];
#pragma unroll
    for (int j = 0; j < ROWS_NW; ++j) wr[j] = w + (size_t)min(n0 + j, N - 1) * K;
    float acc[ROWS_NW][MT];
#pragma unroll
    for (int j = 0; j < ROWS_NW; ++j)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[j][m] = 0.f;
    auto load_w = [&](float4 (&dst)[U][ROWS_NW], int k0) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k = k0 + u * 128 + lane * 4;
#pragma unroll
            for (int j = 0; j < ROWS_NW; ++j) dst[u][j] = k < k_end ? ld_stream(wr[j] + k) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    // The whole block copies the tile's rows (beyond K or M: zeros), asynchronously: a load that the thread
    // itself had to store would hold it for a round trip to the L2 cache before every tile's arithmetic.
    auto load_x = [&](int buf, int k0) {
        for (int i = threadIdx.x; i < MT * (KT / 4); i += ROWS_WARPS * 32) {
            const int m = i / (KT / 4), k = k0 + (i % (KT / 4)) * 4;
            const bool in = m < M && k < k_end;
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(&xs[buf][m][(i % (KT / 4)) * 4]);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(in ? x + (size_t)m * ldx + k : x),
                         "r"(in ? 16 : 0) : "memory");          // 0 bytes read: the 16 bytes are zero-filled
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // the weights do not depend on the kernel before this one: their first tile is requested at once
    float4 wv[U][ROWS_NW];
    load_w(wv, k_lo);
    pdl_wait();
    load_x(0, k_lo);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    int buf = 0;
    for (int k0 = k_lo; k0 < k_end; k0 += KT, buf ^= 1) {
        float4 nx[U][ROWS_NW];
        load_w(nx, k0 + KT);
        if (k0 + KT < k_end) load_x(buf ^ 1, k0 + KT);
#pragma unroll
        for (int u = 0; u < U; ++u) {
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const float4 xv = *reinterpret_cast<const float4*>(&xs[buf][m][u * 128 + lane * 4]);
#pragma unroll
                for (int j = 0; j < ROWS_NW; ++j) {
                    acc[j][m] = fmaf(xv.x, wv[u][j].x, acc[j][m]);
                    acc[j][m] = fmaf(xv.y, wv[u][j].y, acc[j][m]);
                    acc[j][m] = fmaf(xv.z, wv[u][j].z, acc[j][m]);
                    acc[j][m] = fmaf(xv.w, wv[u][j].w, acc[j][m]);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int j = 0; j < ROWS_NW; ++j) wv[u][j] = nx[u][j];
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();      // the next tile's rows are in place, and nobody reads this tile's any more
    }
#pragma unroll
    for (int j = 0; j < ROWS_NW; ++j)
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const float v = warp_sum(acc[j][m]);
            if (lane == 0 && m < M && n0 + j < N) out[(size_t)m * ldo + n0 + j] = v + (bias && blockIdx.y == 0 ? bias[n0 + j] : 0.f);
        }
}

template <int MT>
int launch_rows(const float* x, const float* w, const float* bias, float* out, int M, int N, int K, long long ldx,
                long long ldo, int splits, long long split_stride, cudaStream_t s) {
    const int k_per_split = ((K + splits - 1) / splits + 255) / 256 * 256;       // a multiple of the kernel's k tile
    // (a part that lies wholly beyond K, which the rounding to tiles can leave, is written as zeros)
    RB_LAUNCH((gemm_rows_f32_kernel<MT>), dim3((N + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK, splits), dim3(MT <= 8 ? 128 : 256), 0, s,
              x, w, bias, out, M, N, K, ldx, ldo, k_per_split, split_stride);
    RB_LAUNCH_CHECK();
    return RB_OK;
}

template <typename XT, typename WT, typename OT>
int launch(const void* x, const void* w, const void* bias, void* out, int M, int N, int K, long long ldx,
           long long ldo, cudaStream_t s) {
    if (M > 64 && N > 64) {       // enough rows and columns to fill the large tiles
        dim3 big((N + LBN - 1) / LBN, (M + LBM - 1) / LBM);
        if (big.y > 65535) return RB_ERR_BAD_SIZE;
        RB_LAUNCH((gemm_tn_large_kernel<XT, WT, OT>), dim3(big), dim3(256), 0, s, (const XT*)x, (const WT*)w, (const float*)bias,
                  (OT*)out, M, N, K, ldx, ldo);
        RB_LAUNCH_CHECK();
        return RB_OK;
    }
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
                               int splits, long long split_stride, void* stream) {
    if (M <= 0 || N <= 0) return RB_OK;
    if (K <= 0 || splits < 1) return RB_ERR_BAD_SIZE;
    // splits > 1: float32 partial sums over parts of k at out + z * split_stride (bias in part 0), for the 32-bit
    // product of at most 16 rows only
    if (splits > 1 && !(x_dtype == RB_F32 && w_dtype == RB_F32 && out_dtype == RB_F32 && M <= 16 && K % 4 == 0 &&
                        ldx % 4 == 0 && (((uintptr_t)x | (uintptr_t)w) & 15) == 0))
        return RB_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    typedef __nv_bfloat16 bf;
#define RB_G(XT, WT, OT) return launch<XT, WT, OT>(x, w, bias, out, M, N, K, ldx, ldo, s)
    if (x_dtype == RB_F32 && w_dtype == RB_F32 && out_dtype == RB_F32) {
        // few rows: one pass over the weight (16-byte loads need k, the rows' stride and the pointers to fit)
        if (M <= 16 && K % 4 == 0 && ldx % 4 == 0 && (((uintptr_t)x | (uintptr_t)w) & 15) == 0) {
            const float *xf = (const float*)x, *wf = (const float*)w, *bf32 = (const float*)bias;
            float* of = (float*)out;
            if (M <= 1) return launch_rows<1>(xf, wf, bf32, of, M, N, K, ldx, ldo, splits, split_stride, s);
            if (M <= 2) return launch_rows<2>(xf, wf, bf32, of, M, N, K, ldx, ldo, splits, split_stride, s);
            if (M <= 4) return launch_rows<4>(xf, wf, bf32, of, M, N, K, ldx, ldo, splits, split_stride, s);
            if (M <= 8) return launch_rows<8>(xf, wf, bf32, of, M, N, K, ldx, ldo, splits, split_stride, s);
            return launch_rows<16>(xf, wf, bf32, of, M, N, K, ldx, ldo, splits, split_stride, s);
        }
        RB_G(float, float, float);
    }
    if (x_dtype == RB_F32 && w_dtype == RB_BF16 && out_dtype == RB_F32) RB_G(float, bf, float);
    if (x_dtype == RB_BF16 && w_dtype == RB_BF16 && out_dtype == RB_BF16) RB_G(bf, bf, bf);
    if (x_dtype == RB_BF16 && w_dtype == RB_BF16 && out_dtype == RB_F32) RB_G(bf, bf, float);
    if (x_dtype == RB_BF16 && w_dtype == RB_F32 && out_dtype == RB_BF16) RB_G(bf, float, bf);
    if (x_dtype == RB_BF16 && w_dtype == RB_F32 && out_dtype == RB_F32) RB_G(bf, float, float);
#undef RB_G
    return RB_ERR_BAD_DTYPE;
}
