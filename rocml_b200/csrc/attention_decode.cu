// Decode attention over the paged cache for bfloat16: one query token per sequence, keys split in
// fixed chunks (split-KV), partial results merged by rb_attention_merge.
//
// It is bound by reading the cache once, so the layout serves the loads: a block takes one
// (chunk of 128 keys, key/value head, sequence) and up to 4 query heads of the group, which share
// every key and value it reads.  Inside a warp 8 lanes share a key: each lane holds HD/8
// dimensions of the key row (two 16-byte loads at HD = 128; four adjacent keys make one
// contiguous 1 KB warp load), partial dots are reduced over the 8 lanes with 3 shuffles, and every
// group of 8 lanes keeps its own running maximum, sum and accumulator for the keys it saw.  The
// 16 groups of the block are merged once at the end through shared memory.  Softmax statistics and
// accumulators are float32; exp is expf.
//
// Replaces attn_decode_partial_f16 of the reference (rocml-kernels/kernels/attn_decode.hip:93-211):
// same mathematics (head h reads key/value head h / g, score = (q.k) * scale, online max/sum,
// unnormalised partial result per split), other mapping.  Head sizes 64, 128 and 256; other sizes
// use the plain kernel.
#include "common.cuh"
#include "api.h"

using namespace rb;

namespace {
constexpr int CHUNK = 128;        // keys per block
constexpr int WARPS = 4;
constexpr int KEYS_PER_ITER = 4;  // per warp: 32 lanes / 8 lanes per key
constexpr float NEG_BIG = -1e30f;

struct alignas(16) Pack8 { __nv_bfloat162 v[4]; };  // 8 bf16 = 16 bytes

template <int HD, int GC>
__global__ void __launch_bounds__(WARPS * 32)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, int q_stride,
                        const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                        const int* __restrict__ block_table, int max_pages, const int* __restrict__ seq_slot,
                        const int* __restrict__ cu_q, const int* __restrict__ kv_len, int nq, int nkv,
                        float scale, int window, int n_chunks, float* __restrict__ part_acc,
                        float* __restrict__ part_ml, __nv_bfloat16* __restrict__ out, int o_stride) {
    constexpr int DPL = HD / 8;          // dimensions per lane
    constexpr int VEC = DPL / 8;         // 16-byte loads per lane per row
    const int c = blockIdx.x;
    const int g = nq / nkv;
    const int head_chunks = g / GC;
    const int kvh = blockIdx.y / head_chunks;
    const int h0 = kvh * g + (blockIdx.y % head_chunks) * GC;   // first query head of this block
    const int b = blockIdx.z;
    const int slot = seq_slot[b];
    if (slot < 0) return;
    const int t = cu_q[b];
    const int pos = kv_len[b] - 1;
    const int lo = max(window > 0 ? max(0, pos - window + 1) : 0, c * CHUNK);
    const int hi = min(pos, (c + 1) * CHUNK - 1);
    if (c * CHUNK > pos) return;         // never merged

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane & 7, grp = lane >> 3;
    const int* table = block_table + (size_t)slot * max_pages;

    // this lane's slice of the query heads, as float
    float qf[GC][DPL];
#pragma unroll
    for (int h = 0; h < GC; ++h) {
        const __nv_bfloat16* qp = q + (size_t)t * q_stride + (size_t)(h0 + h) * HD + sub * DPL;
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
            const Pack8 pk = *reinterpret_cast<const Pack8*>(qp + v * 8);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(pk.v[i]);
                qf[h][v * 8 + 2 * i] = f.x;
                qf[h][v * 8 + 2 * i + 1] = f.y;
            }
        }
    }
    float m[GC], l[GC], acc[GC][DPL];
#pragma unroll
    for (int h = 0; h < GC; ++h) {
        m[h] = NEG_BIG;
        l[h] = 0.f;
#pragma unroll
        for (int d = 0; d < DPL; ++d) acc[h][d] = 0.f;
    }

    // keys of this chunk: warp w, iteration it, group grp -> key c*CHUNK + (it*WARPS + w)*4 + grp
    constexpr int ITERS = CHUNK / (WARPS * KEYS_PER_ITER);
#pragma unroll 2
    for (int it = 0; it < ITERS; ++it) {
        const int j = c * CHUNK + (it * WARPS + warp) * KEYS_PER_ITER + grp;
        const bool valid = j >= lo && j <= hi;
        Pack8 kk[VEC], vv[VEC];
        if (valid) {
            const int page = table[j / RB_PAGE];
            const size_t off = (((size_t)page * nkv + kvh) * RB_PAGE + (j % RB_PAGE)) * HD + sub * DPL;
#pragma unroll
            for (int v = 0; v < VEC; ++v) {
                kk[v] = *reinterpret_cast<const Pack8*>(k_cache + off + v * 8);
                vv[v] = *reinterpret_cast<const Pack8*>(v_cache + off + v * 8);
            }
        } else {
#pragma unroll
            for (int v = 0; v < VEC; ++v) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    kk[v].v[i] = __float2bfloat162_rn(0.f);
                    vv[v].v[i] = __float2bfloat162_rn(0.f);
                }
            }
        }
        float kf[DPL], vf[DPL];
#pragma unroll
        for (int v = 0; v < VEC; ++v)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 a = __bfloat1622float2(kk[v].v[i]);
                const float2 bb = __bfloat1622float2(vv[v].v[i]);
                kf[v * 8 + 2 * i] = a.x; kf[v * 8 + 2 * i + 1] = a.y;
                vf[v * 8 + 2 * i] = bb.x; vf[v * 8 + 2 * i + 1] = bb.y;
            }
#pragma unroll
        for (int h = 0; h < GC; ++h) {
            float s = 0.f;
#pragma unroll
            for (int d = 0; d < DPL; ++d) s = fmaf(qf[h][d], kf[d], s);
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            s += __shfl_xor_sync(0xffffffffu, s, 4);
            s *= scale;   // after the dot, as the reference does
            if (valid) {
                const float m_new = fmaxf(m[h], s);
                const float alpha = expf(m[h] - m_new);
                const float p = expf(s - m_new);
                l[h] = l[h] * alpha + p;
                m[h] = m_new;
#pragma unroll
                for (int d = 0; d < DPL; ++d) acc[h][d] = fmaf(p, vf[d], acc[h][d] * alpha);
            }
        }
    }

    // merge the 16 groups (4 per warp x 4 warps) of the block through shared memory
    __shared__ float s_m[WARPS * 4][GC], s_l[WARPS * 4][GC];
    __shared__ float s_acc[WARPS * 4][GC][HD + 4];
    const int gi = warp * 4 + grp;
#pragma unroll
    for (int h = 0; h < GC; ++h) {
        if (sub == 0) { s_m[gi][h] = m[h]; s_l[gi][h] = l[h]; }
#pragma unroll
        for (int d = 0; d < DPL; ++d) s_acc[gi][h][sub * DPL + d] = acc[h][d];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < GC * HD; idx += WARPS * 32) {
        const int h = idx / HD, d = idx % HD;
        float M = NEG_BIG;
#pragma unroll
        for (int i = 0; i < WARPS * 4; ++i) M = fmaxf(M, s_m[i][h]);
        float L = 0.f, A = 0.f;
#pragma unroll
        for (int i = 0; i < WARPS * 4; ++i) {
            const float w = expf(s_m[i][h] - M);     // groups that saw nothing have l = 0, acc = 0
            L = fmaf(w, s_l[i][h], L);
            A = fmaf(w, s_acc[i][h][d], A);
        }
        const int head = h0 + h;
        if (n_chunks > 1) {
            const size_t pidx = ((size_t)t * nq + head) * n_chunks + c;
            part_acc[pidx * HD + d] = A;
            if (d == 0) { part_ml[pidx * 2] = M; part_ml[pidx * 2 + 1] = L; }
        } else {
            out[(size_t)t * o_stride + (size_t)head * HD + d] = __float2bfloat16_rn(L > 0.f ? A / L : 0.f);
        }
    }
}

template <int HD, int GC>
int launch(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int* block_table,
           int max_pages, const int* seq_slot, const int* cu_q, const int* kv_len, int B, int nq, int nkv,
           float scale, int window, int n_chunks, float* part_acc, float* part_ml, void* out, int o_stride,
           cudaStream_t s) {
    const int g = nq / nkv;
    dim3 grid(n_chunks, nkv * (g / GC), B);
    if (grid.y > 65535 || grid.z > 65535) return RB_ERR_BAD_SIZE;
    attention_decode_kernel<HD, GC><<<grid, WARPS * 32, 0, s>>>(
        (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
        block_table, max_pages, seq_slot, cu_q, kv_len, nq, nkv, scale, window, n_chunks, part_acc, part_ml,
        (__nv_bfloat16*)out, o_stride);
    RB_LAUNCH_CHECK();
    return RB_OK;
}
}  // namespace

// One query token per sequence (token index cu_q[b]).  chunk is fixed at 128 keys; n_chunks covers
// the longest sequence of the batch; with n_chunks == 1 the result is written to `out` directly.
// Returns RB_ERR_BAD_SIZE for head sizes other than 64, 128, 256 (the caller uses the plain kernel).
extern "C" int rb_attention_decode(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                   const int* block_table, int max_pages, const int* seq_slot, const int* cu_q,
                                   const int* kv_len, int B, int nq, int nkv, int hd, float scale, int window,
                                   int n_chunks, float* part_acc, float* part_ml, void* out, int o_stride,
                                   void* stream) {
    if (B <= 0) return RB_OK;
    if (nkv <= 0 || nq % nkv || n_chunks < 1) return RB_ERR_BAD_SIZE;
    if (((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15) || (q_stride % 8))
        return RB_ERR_BAD_ALIGN;
    cudaStream_t s = (cudaStream_t)stream;
    const int g = nq / nkv;
    const int gc = g % 4 == 0 ? 4 : (g % 2 == 0 ? 2 : 1);
#define RB_AD(HD, GC) return launch<HD, GC>(q, q_stride, k_cache, v_cache, block_table, max_pages, seq_slot, cu_q, \
                                            kv_len, B, nq, nkv, scale, window, n_chunks, part_acc, part_ml, out, o_stride, s)
    if (hd == 128) { if (gc == 4) RB_AD(128, 4); if (gc == 2) RB_AD(128, 2); RB_AD(128, 1); }
    if (hd == 64) { if (gc == 4) RB_AD(64, 4); if (gc == 2) RB_AD(64, 2); RB_AD(64, 1); }
    if (hd == 256) { if (gc == 4) RB_AD(256, 2); if (gc == 2) RB_AD(256, 2); RB_AD(256, 1); }
#undef RB_AD
    return RB_ERR_BAD_SIZE;
}
