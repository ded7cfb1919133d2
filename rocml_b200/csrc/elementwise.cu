// Embedding gather, fused residual-add + RMSNorm, SiLU(gate) * up, casts.
//
// All arithmetic is 32-bit; only loads and stores use the storage types.
#include "common.cuh"
#include "api.h"

using namespace rb;

// ---- embedding: resid[t, :] = f32(table[ids[t], :]) --------------------------------------
// Replaces the reference's embedding_f16_f32 (rocml-kernels/kernels/embedding.hip:6-18).
template <typename WT>
__global__ void embedding_kernel(const int* __restrict__ ids, const WT* __restrict__ table,
                                 float* __restrict__ out, int H, int vocab, int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * H;
    if (id < 0 || id >= vocab) {  // a token id outside the table: record it, write zeros
        if (threadIdx.x == 0 && status) atomicExch(status, RB_ERR_BAD_SIZE);
        for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const WT* row = table + (size_t)id * H;
    if (sizeof(WT) == 2 && H % 8 == 0 && (((uintptr_t)table | (uintptr_t)out) & 15) == 0) {
        // 16 bytes a load, and a thread's loads all requested before the first is used: a row of a table of a
        // gigabyte comes from memory, and loads taken one after the other would each wait for it
        constexpr int UNROLL = 4;
        const int n8 = H / 8;
        for (int i0 = threadIdx.x; i0 < n8; i0 += blockDim.x * UNROLL) {
            uint4 raw[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int i = i0 + u * blockDim.x;
                raw[u] = i < n8 ? reinterpret_cast<const uint4*>(row)[i] : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int i = i0 + u * blockDim.x;
                if (i >= n8) continue;
                const uint32_t ws[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
                float4 lo, hi;
                lo.x = __uint_as_float(ws[0] << 16); lo.y = __uint_as_float(ws[0] & 0xFFFF0000u);
                lo.z = __uint_as_float(ws[1] << 16); lo.w = __uint_as_float(ws[1] & 0xFFFF0000u);
                hi.x = __uint_as_float(ws[2] << 16); hi.y = __uint_as_float(ws[2] & 0xFFFF0000u);
                hi.z = __uint_as_float(ws[3] << 16); hi.w = __uint_as_float(ws[3] & 0xFFFF0000u);
                reinterpret_cast<float4*>(o)[2 * i] = lo;
                reinterpret_cast<float4*>(o)[2 * i + 1] = hi;
            }
        }
        return;
    }
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_f32(row[i]);
}

extern "C" int rb_embedding(const int* ids, const void* table, int table_dtype, float* out, int T,
                            int H, int vocab, int* status, void* stream) {
    if (T <= 0) return RB_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_dtype == RB_BF16)
        RB_LAUNCH((embedding_kernel<__nv_bfloat16>), dim3(T), dim3(threads), 0, s, ids, (const __nv_bfloat16*)table, out, H, vocab, status);
    else if (table_dtype == RB_F32)
        RB_LAUNCH((embedding_kernel<float>), dim3(T), dim3(threads), 0, s, ids, (const float*)table, out, H, vocab, status);
    else
        return RB_ERR_BAD_DTYPE;
    RB_LAUNCH_CHECK();
    return RB_OK;
}

// ---- fused residual add + RMSNorm ---------------------------------------------------------
// r = resid[row] + sum_s delta[s][row]   (s in fixed order, so the sum never depends on the batch)
// if write_back: resid[row] = r
// out[i] = r * rsqrt(mean(r^2) + eps) * w
// `rows` (optional) picks the source rows; output row i is compact.  One block per output row.
// Replaces add_inplace_f32 + rmsnorm_f32 (rocml-kernels/kernels/elementwise.hip:7-26,
// rmsnorm.hip:7-43); product order x * inv_rms * w as there.
// Four consecutive outputs: one 8- or 16-byte store when the row allows it.
__device__ __forceinline__ void store4(float* p, float a, float b, float c, float d, bool vec) {
    if (vec) *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
    else { p[0] = a; p[1] = b; p[2] = c; p[3] = d; }
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, float a, float b, float c, float d, bool vec) {
    if (vec) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t*>(&lo);
        raw.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p) = raw;
    } else {
        p[0] = __float2bfloat16_rn(a); p[1] = __float2bfloat16_rn(b);
        p[2] = __float2bfloat16_rn(c); p[3] = __float2bfloat16_rn(d);
    }
}

template <typename OT, typename WT>
__global__ void __launch_bounds__(1024) add_rmsnorm_kernel(float* __restrict__ resid, const float* __restrict__ delta,
                                   int n_delta, size_t delta_stride, const WT* __restrict__ w,
                                   OT* __restrict__ out, const int* __restrict__ rows, int H,
                                   float eps, int write_back) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float row_buf[];  // H floats (padded to 4) + 33 for the reduction
    float* red = row_buf + ((H + 3) & ~3);
    const int orow = blockIdx.x;
    const int row = rows ? rows[orow] : orow;
    if (row < 0) return;  // a padded entry
    float* r = resid + (size_t)row * H;
    float ss = 0.f;
    const bool vec = (H & 3) == 0 && (delta_stride & 3) == 0 && (((uintptr_t)resid | (uintptr_t)delta) & 15) == 0;
    if (vec) {
        const int H4 = H >> 2;
        float4* rb4 = reinterpret_cast<float4*>(row_buf);
        const float4* r4 = reinterpret_cast<const float4*>(r);
        for (int i = threadIdx.x; i < H4; i += blockDim.x) {
            float4 v = r4[i];
            const float4* d4 = reinterpret_cast<const float4*>(delta + (size_t)row * H) + i;
            const size_t ds4 = delta_stride >> 2;
            // eight partial sums at a time: every load is issued before the first addition, and the
            // additions keep the partial sums' order (an absent one adds zero)
            for (int s = 0; s < n_delta; s += 8) {
                float4 d[8];
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    d[j] = s + j < n_delta ? d4[(size_t)(s + j) * ds4] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int j = 0; j < 8; ++j) { v.x += d[j].x; v.y += d[j].y; v.z += d[j].z; v.w += d[j].w; }
            }
            rb4[i] = v;
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            float v = r[i];
            for (int s = 0; s < n_delta; ++s) v += delta[(size_t)s * delta_stride + (size_t)row * H + i];
            row_buf[i] = v;
            ss += v * v;
        }
    }
    const float total = block_sum(ss, red);
    const float inv = rsqrtf(total / (float)H + eps);
    OT* o = out + (size_t)orow * H;
    const bool out_vec = (((uintptr_t)out | ((size_t)H * sizeof(OT))) & 15) == 0;
    if (vec) {
        const int H4 = H >> 2;
        const float4* rb4 = reinterpret_cast<const float4*>(row_buf);
        float4* r4 = reinterpret_cast<float4*>(r);
        for (int i = threadIdx.x; i < H4; i += blockDim.x) {
            const float4 v = rb4[i];
            if (write_back) r4[i] = v;
            store4(o + 4 * i, v.x * inv * to_f32(w[4 * i]), v.y * inv * to_f32(w[4 * i + 1]),
                   v.z * inv * to_f32(w[4 * i + 2]), v.w * inv * to_f32(w[4 * i + 3]), out_vec);
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            const float v = row_buf[i];
            if (write_back) r[i] = v;
            o[i] = from_f32<OT>(v * inv * to_f32(w[i]));
        }
    }
}

// The same for many rows (prompts): a row per block of 128 or 256 threads, each thread keeping up to
// eight 16-byte groups of the row in registers, so that the row is read once, all its loads are in
// flight together, and several rows share a multiprocessor.  Needs 16-byte alignment throughout and
// H <= 8 * 4 * threads.
template <typename OT, typename WT, int THREADS>
__global__ void __launch_bounds__(THREADS) add_rmsnorm_rows_kernel(float* __restrict__ resid, const float* __restrict__ delta,
                                                                   int n_delta, size_t delta_stride,
                                                                   const WT* __restrict__ w, OT* __restrict__ out,
                                                                   const int* __restrict__ rows, int H, float eps,
                                                                   int write_back) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[33];
    const int orow = blockIdx.x;
    const int row = rows ? rows[orow] : orow;
    if (row < 0) return;  // a padded entry
    const int H4 = H >> 2;
    float4* r4 = reinterpret_cast<float4*>(resid + (size_t)row * H);
    float4 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = threadIdx.x + j * THREADS;
        v[j] = i < H4 ? r4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int s = 0; s < n_delta; s += 2) {                  // partial sums in their order, two in flight
        const float4* d4 = reinterpret_cast<const float4*>(delta + (size_t)s * delta_stride + (size_t)row * H);
        const float4* e4 = reinterpret_cast<const float4*>(delta + (size_t)(s + 1) * delta_stride + (size_t)row * H);
        const bool second = s + 1 < n_delta;
        float4 d[8], e[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = threadIdx.x + j * THREADS;
            d[j] = i < H4 ? d4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            e[j] = second && i < H4 ? e4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) { v[j].x += d[j].x; v[j].y += d[j].y; v[j].z += d[j].z; v[j].w += d[j].w; }
#pragma unroll
        for (int j = 0; j < 8; ++j) { v[j].x += e[j].x; v[j].y += e[j].y; v[j].z += e[j].z; v[j].w += e[j].w; }
    }
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
    const float inv = rsqrtf(block_sum(ss, red) / (float)H + eps);
    OT* o = out + (size_t)orow * H;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = threadIdx.x + j * THREADS;
        if (i < H4) {
            if (write_back) r4[i] = v[j];
            store4(o + 4 * i, v[j].x * inv * to_f32(w[4 * i]), v[j].y * inv * to_f32(w[4 * i + 1]),
                   v[j].z * inv * to_f32(w[4 * i + 2]), v[j].w * inv * to_f32(w[4 * i + 3]), true);
        }
    }
}

template <typename OT, typename WT>
static int launch_add_rmsnorm(float* resid, const float* delta, int n_delta, size_t delta_stride,
                              const void* w, void* out, const int* rows, int n_rows, int H, float eps,
                              int write_back, cudaStream_t s) {
    // many rows: the register kernel, when everything is 16-byte aligned and a row fits its threads
    // (up to 256 rows are at most one wave of the kernel below, whose 1,024 threads a row finish sooner)
    const bool aligned = (H & 3) == 0 && (delta_stride & 3) == 0 &&
                         ((((uintptr_t)resid | (uintptr_t)delta) & 15) == 0) &&
                         ((((uintptr_t)out | ((size_t)H * sizeof(OT))) & 15) == 0) && (((uintptr_t)w & (4 * sizeof(WT) - 1)) == 0);
    if (n_rows > (H >= 4096 ? 256 : 64) && aligned && H <= 8 * 4 * 256) {
        if (H <= 8 * 4 * 128)
            RB_LAUNCH((add_rmsnorm_rows_kernel<OT, WT, 128>), dim3(n_rows), dim3(128), 0, s, resid, delta, n_delta,
                      delta_stride, (const WT*)w, (OT*)out, rows, H, eps, write_back);
        else
            RB_LAUNCH((add_rmsnorm_rows_kernel<OT, WT, 256>), dim3(n_rows), dim3(256), 0, s, resid, delta, n_delta,
                      delta_stride, (const WT*)w, (OT*)out, rows, H, eps, write_back);
        RB_LAUNCH_CHECK();
        return RB_OK;
    }
    const size_t smem = (size_t)(((H + 3) & ~3) + 33) * sizeof(float);
    if (smem > 200 * 1024) return RB_ERR_BAD_SIZE;
    auto k = add_rmsnorm_kernel<OT, WT>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    // one 16-byte column group per thread where the row allows it: a row's loads are all in flight at once
    const int threads = H >= 4096 ? 1024 : (H >= 2048 ? 512 : (H >= 512 ? 256 : 128));
    RB_LAUNCH((k), dim3(n_rows), dim3(threads), smem, s, resid, delta, n_delta, delta_stride, (const WT*)w, (OT*)out, rows, H,
                                    eps, write_back);
    RB_LAUNCH_CHECK();
    return RB_OK;
}

extern "C" int rb_add_rmsnorm(float* resid, const float* delta, int n_delta, long long delta_stride,
                              const void* w, int w_dtype, void* out, int out_dtype, const int* rows,
                              int n_rows, int H, float eps, int write_back, void* stream) {
    if (n_rows <= 0) return RB_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t ds = (size_t)delta_stride;
    if (out_dtype == RB_BF16 && w_dtype == RB_BF16)
        return launch_add_rmsnorm<__nv_bfloat16, __nv_bfloat16>(resid, delta, n_delta, ds, w, out, rows, n_rows, H, eps, write_back, s);
    if (out_dtype == RB_BF16 && w_dtype == RB_F32)
        return launch_add_rmsnorm<__nv_bfloat16, float>(resid, delta, n_delta, ds, w, out, rows, n_rows, H, eps, write_back, s);
    if (out_dtype == RB_F32 && w_dtype == RB_BF16)
        return launch_add_rmsnorm<float, __nv_bfloat16>(resid, delta, n_delta, ds, w, out, rows, n_rows, H, eps, write_back, s);
    if (out_dtype == RB_F32 && w_dtype == RB_F32)
        return launch_add_rmsnorm<float, float>(resid, delta, n_delta, ds, w, out, rows, n_rows, H, eps, write_back, s);
    return RB_ERR_BAD_DTYPE;
}

// ---- SiLU(gate) * up ------------------------------------------------------------------------
// in: [S][T, 2*I] (S partial sums that are added first, in order); out: [T, I].  The gate of output
// i sits in column i and its up in column I + i, or, when `paired`, columns alternate in blocks of
// 16 between gates and ups (gate of output i at (i / 16) * 32 + i % 16, its up 16 columns on).  silu(g) = g / (1 + exp(-g)) as in
// rocml-kernels/kernels/silu_mul.hip:15-18.  Four outputs per thread when I is a multiple of 4.
template <typename IT, typename OT>
__global__ void silu_mul_kernel(const IT* __restrict__ in, int n_in, size_t in_stride, OT* __restrict__ out,
                                int rows, int I, int paired) {
    pdl_trigger();
    pdl_wait();
    const int I4 = I >> 2;
    const bool vec = (I & 3) == 0;
    const bool in16 = ((uintptr_t)in & 15) == 0 && (in_stride & 3) == 0;     // with I a multiple of 4: every group of 4 on 16 bytes
    const size_t n = vec ? (size_t)rows * I4 : (size_t)rows * I;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
         idx += (size_t)gridDim.x * blockDim.x) {
        if (vec) {
            const size_t t = idx / I4;
            const int i = (int)(idx - t * I4) * 4;
            float g[4] = {0.f, 0.f, 0.f, 0.f}, u[4] = {0.f, 0.f, 0.f, 0.f};
            const int gi = paired ? (i >> 4) * 32 + (i & 15) : i;
            const int up = paired ? 16 : I;
            if (sizeof(IT) == 4 && in16) {
                // 16-byte loads, two partial sums' worth in flight together; added in the partial sums' order
                for (int s = 0; s < n_in; s += 2) {
                    const float* p = reinterpret_cast<const float*>(in) + (size_t)s * in_stride + t * 2 * I + gi;
                    const bool second = s + 1 < n_in;
                    const float4 g0 = *reinterpret_cast<const float4*>(p), u0 = *reinterpret_cast<const float4*>(p + up);
                    const float4 g1 = second ? *reinterpret_cast<const float4*>(p + in_stride) : make_float4(0.f, 0.f, 0.f, 0.f);
                    const float4 u1 = second ? *reinterpret_cast<const float4*>(p + in_stride + up) : make_float4(0.f, 0.f, 0.f, 0.f);
                    g[0] += g0.x; g[1] += g0.y; g[2] += g0.z; g[3] += g0.w;
                    u[0] += u0.x; u[1] += u0.y; u[2] += u0.z; u[3] += u0.w;
                    g[0] += g1.x; g[1] += g1.y; g[2] += g1.z; g[3] += g1.w;
                    u[0] += u1.x; u[1] += u1.y; u[2] += u1.z; u[3] += u1.w;
                }
            } else {
                for (int s = 0; s < n_in; ++s) {
                    const IT* p = in + (size_t)s * in_stride + t * 2 * I + gi;
#pragma unroll
                    for (int j = 0; j < 4; ++j) { g[j] += to_f32(p[j]); u[j] += to_f32(p[up + j]); }
                }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) out[t * I + i + j] = from_f32<OT>(g[j] / (1.f + expf(-g[j])) * u[j]);
        } else {
            const size_t t = idx / I;
            const int i = (int)(idx - t * I);
            float g = 0.f, u = 0.f;
            for (int s = 0; s < n_in; ++s) {
                const int gi = paired ? (i >> 4) * 32 + (i & 15) : i;
                g += to_f32(in[(size_t)s * in_stride + t * 2 * I + gi]);
                u += to_f32(in[(size_t)s * in_stride + t * 2 * I + gi + (paired ? 16 : I)]);
            }
            out[idx] = from_f32<OT>(g / (1.f + expf(-g)) * u);
        }
    }
}

extern "C" int rb_silu_mul(const void* in, int in_dtype, int n_in, long long in_stride, void* out, int out_dtype,
                           int rows, int I, int paired, void* stream) {
    if (rows <= 0) return RB_OK;
    if (n_in < 1 || (paired && I % 16)) return RB_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t n = (I & 3) == 0 ? (size_t)rows * (I >> 2) : (size_t)rows * I;
    const int threads = 256;
    const size_t want = (n + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 32 ? want : 148 * 32);
    typedef __nv_bfloat16 bf;
    if (in_dtype == RB_BF16 && out_dtype == RB_BF16)
        RB_LAUNCH((silu_mul_kernel<bf, bf>), dim3(blocks), dim3(threads), 0, s, (const bf*)in, n_in, (size_t)in_stride, (bf*)out, rows, I, paired);
    else if (in_dtype == RB_F32 && out_dtype == RB_BF16)
        RB_LAUNCH((silu_mul_kernel<float, bf>), dim3(blocks), dim3(threads), 0, s, (const float*)in, n_in, (size_t)in_stride, (bf*)out, rows, I, paired);
    else if (in_dtype == RB_F32 && out_dtype == RB_F32)
        RB_LAUNCH((silu_mul_kernel<float, float>), dim3(blocks), dim3(threads), 0, s, (const float*)in, n_in, (size_t)in_stride, (float*)out, rows, I, paired);
    else
        return RB_ERR_BAD_DTYPE;
    return RB_OK;
}

// ---- casts ------------------------------------------------------------------------------------
template <typename A, typename B>
__global__ void cast_kernel(const A* __restrict__ in, B* __restrict__ out, size_t n) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_f32<B>(to_f32(in[i]));
}

extern "C" int rb_cast(const void* in, int in_dtype, void* out, int out_dtype, long long n, void* stream) {
    if (n <= 0) return RB_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 256;
    const long long want = (n + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    if (in_dtype == RB_F32 && out_dtype == RB_BF16)
        RB_LAUNCH((cast_kernel<float, __nv_bfloat16>), dim3(blocks), dim3(threads), 0, s, (const float*)in, (__nv_bfloat16*)out, (size_t)n);
    else if (in_dtype == RB_BF16 && out_dtype == RB_F32)
        RB_LAUNCH((cast_kernel<__nv_bfloat16, float>), dim3(blocks), dim3(threads), 0, s, (const __nv_bfloat16*)in, (float*)out, (size_t)n);
    else
        return RB_ERR_BAD_DTYPE;
    RB_LAUNCH_CHECK();
    return RB_OK;
}
