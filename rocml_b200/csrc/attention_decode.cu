// Decode attention over the paged cache for bfloat16: one query token per sequence, keys split in
// fixed chunks of 128 (split-KV), the chunks' partial results merged by the block that finishes last.
//
// It is bound by reading the cache once, so the layout serves the loads: a block of 8 warps takes
// one (chunk, key/value head, sequence) and up to 4 query heads of the group, which share every key
// and value it reads.  Inside a warp 8 lanes share a key: each lane holds HD/8 dimensions of the
// key row (two 16-byte loads at HD = 128; four adjacent keys make one contiguous 1 KB warp load).
// Every thread first issues ALL its loads (4 keys and 4 values), then computes: partial dots are
// reduced over the 8 lanes with 3 shuffles, each group of 8 lanes forms the softmax statistics of
// its own 4 keys, and the 32 groups of the block are merged through shared memory.  The block
// writes an unnormalised partial result; a counter per (sequence, head group) tells the last block
// to arrive, which merges all chunks in ascending order and writes the output (the counter is left
// at zero for the next launch).  Statistics and accumulators are float32; exp is expf.
//
// Replaces attn_decode_partial_f16 + attn_decode_reduce_f32 of the reference
// (rocml-kernels/kernels/attn_decode.hip:93-255): same mathematics (head h reads key/value head
// h / g, score = (q.k) * scale, max/sum softmax, split over the keys, log-sum-exp merge), other
// mapping.  Head sizes 64, 128 and 256; other sizes use the plain kernel.
#include "common.cuh"
#include "api.h"

using namespace rb;

namespace {
constexpr int CHUNK = 128;        // keys per block
constexpr int WARPS = 8;
constexpr int KPT = CHUNK / (WARPS * 4);   // keys per 8-lane group: 4
constexpr float NEG_BIG = -1e30f;

struct alignas(16) Pack8 { __nv_bfloat162 v[4]; };  // 8 bf16 = 16 bytes

template <int HD, int GC>
__global__ void __launch_bounds__(WARPS * 32)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, int q_stride,
                        const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                        const int* __restrict__ block_table, int max_pages, const int* __restrict__ seq_slot,
                        const int* __restrict__ cu_q, const int* __restrict__ kv_len, int nq, int nkv,
                        float scale, int window, int n_chunks, float* __restrict__ part_acc,
                        float* __restrict__ part_ml, int* __restrict__ counters,
                        __nv_bfloat16* __restrict__ out, int o_stride) {
    pdl_trigger();
    pdl_wait();
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
    if (c * CHUNK > pos) return;         // beyond the sequence: takes no part in the merge
    const int lo = max(window > 0 ? max(0, pos - window + 1) : 0, c * CHUNK);
    const int hi = min(pos, (c + 1) * CHUNK - 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane & 7, grp = lane >> 3;
    const int* table = block_table + (size_t)slot * max_pages;

    // all loads first: this group's keys are j0 + i * 32 (i < KPT), so that at every i the block
    // reads 32 adjacent keys
    const int j0 = c * CHUNK + warp * 4 + grp;
    Pack8 kk[KPT][VEC], vv[KPT][VEC];
    bool valid[KPT];
#pragma unroll
    for (int i = 0; i < KPT; ++i) {
        const int j = j0 + i * 32;
        valid[i] = j >= lo && j <= hi;
        if (valid[i]) {
            const int page = table[j / RB_PAGE];
            const size_t off = (((size_t)page * nkv + kvh) * RB_PAGE + (j % RB_PAGE)) * HD + sub * DPL;
#pragma unroll
            for (int v = 0; v < VEC; ++v) {
                kk[i][v] = *reinterpret_cast<const Pack8*>(k_cache + off + v * 8);
                vv[i][v] = *reinterpret_cast<const Pack8*>(v_cache + off + v * 8);
            }
        } else {
#pragma unroll
            for (int v = 0; v < VEC; ++v)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    kk[i][v].v[e] = __float2bfloat162_rn(0.f);
                    vv[i][v].v[e] = __float2bfloat162_rn(0.f);
                }
        }
    }
    // this lane's slice of the query heads
    float qf[GC][DPL];
#pragma unroll
    for (int h = 0; h < GC; ++h) {
        const __nv_bfloat16* qp = q + (size_t)t * q_stride + (size_t)(h0 + h) * HD + sub * DPL;
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
            const Pack8 pk = *reinterpret_cast<const Pack8*>(qp + v * 8);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(pk.v[e]);
                qf[h][v * 8 + 2 * e] = f.x;
                qf[h][v * 8 + 2 * e + 1] = f.y;
            }
        }
    }
    // scores of this group's keys
    float sc[KPT][GC];
#pragma unroll
    for (int i = 0; i < KPT; ++i) {
#pragma unroll
        for (int h = 0; h < GC; ++h) {
            float s = 0.f;
#pragma unroll
            for (int v = 0; v < VEC; ++v)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 kf = __bfloat1622float2(kk[i][v].v[e]);
                    s = fmaf(qf[h][v * 8 + 2 * e], kf.x, s);
                    s = fmaf(qf[h][v * 8 + 2 * e + 1], kf.y, s);
                }
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            s += __shfl_xor_sync(0xffffffffu, s, 4);
            sc[i][h] = valid[i] ? s * scale : NEG_BIG;   // scale after the dot, as the reference does
        }
    }
    // softmax statistics and weighted values of the group's keys
    __shared__ float s_m[WARPS * 4][GC], s_l[WARPS * 4][GC];
    __shared__ float s_acc[WARPS][GC][HD + 4];
    __shared__ int s_last;
    float m[GC], l[GC], acc[GC][DPL];
#pragma unroll
    for (int h = 0; h < GC; ++h) {
        m[h] = NEG_BIG;
#pragma unroll
        for (int i = 0; i < KPT; ++i) m[h] = fmaxf(m[h], sc[i][h]);
        l[h] = 0.f;
#pragma unroll
        for (int d = 0; d < DPL; ++d) acc[h][d] = 0.f;
    }
#pragma unroll
    for (int i = 0; i < KPT; ++i) {
        float vf[DPL];
#pragma unroll
        for (int v = 0; v < VEC; ++v)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(vv[i][v].v[e]);
                vf[v * 8 + 2 * e] = f.x;
                vf[v * 8 + 2 * e + 1] = f.y;
            }
#pragma unroll
        for (int h = 0; h < GC; ++h) {
            const float p = valid[i] ? expf(sc[i][h] - m[h]) : 0.f;
            l[h] += p;
#pragma unroll
            for (int d = 0; d < DPL; ++d) acc[h][d] = fmaf(p, vf[d], acc[h][d]);
        }
    }
    // block maximum per head, then every group rescales its own sums to it
    const int gi = warp * 4 + grp;
    if (sub == 0) {
#pragma unroll
        for (int h = 0; h < GC; ++h) s_m[gi][h] = m[h];
    }
    __syncthreads();
    float M[GC];
#pragma unroll
    for (int h = 0; h < GC; ++h) {
        float mm = NEG_BIG;
        for (int i = 0; i < WARPS * 4; ++i) mm = fmaxf(mm, s_m[i][h]);
        M[h] = mm;
        const float w = expf(m[h] - mm);      // a group that saw no key has l = 0 and acc = 0
        l[h] *= w;
#pragma unroll
        for (int d = 0; d < DPL; ++d) acc[h][d] *= w;
        // the 4 groups of the warp are added with shuffles, the 8 warps through shared memory
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 8);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 16);
#pragma unroll
        for (int d = 0; d < DPL; ++d) {
            acc[h][d] += __shfl_xor_sync(0xffffffffu, acc[h][d], 8);
            acc[h][d] += __shfl_xor_sync(0xffffffffu, acc[h][d], 16);
        }
        if (grp == 0) {
            if (sub == 0) s_l[warp][h] = l[h];
#pragma unroll
            for (int d = 0; d < DPL; ++d) s_acc[warp][h][sub * DPL + d] = acc[h][d];
        }
    }
    __syncthreads();

    const size_t row = (size_t)t * nq;
    for (int idx = threadIdx.x; idx < GC * HD; idx += WARPS * 32) {
        const int h = idx / HD, d = idx % HD;
        float L = 0.f, A = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) { L += s_l[w][h]; A += s_acc[w][h][d]; }
        const int head = h0 + h;
        if (n_chunks > 1) {
            const size_t pidx = (row + head) * n_chunks + c;
            part_acc[pidx * HD + d] = A;
            if (d == 0) {
                float mm = NEG_BIG;
                for (int i = 0; i < WARPS * 4; ++i) mm = fmaxf(mm, s_m[i][h]);
                part_ml[pidx * 2] = mm;
                part_ml[pidx * 2 + 1] = L;
            }
        } else {
            out[(size_t)t * o_stride + (size_t)head * HD + d] = __float2bfloat16_rn(L > 0.f ? A / L : 0.f);
        }
    }
    if (n_chunks <= 1) return;

    // the block that arrives last merges the chunks of this (sequence, head group)
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int active = pos / CHUNK + 1;
        int* ctr = counters + (size_t)b * gridDim.y + blockIdx.y;
        const int old = atomicAdd(ctr, 1);
        s_last = old == active - 1;
        if (s_last) *ctr = 0;              // ready for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const int c_hi = pos / CHUNK;
    const int c_lo = window > 0 ? max(0, pos - window + 1) / CHUNK : 0;
    for (int idx = threadIdx.x; idx < GC * HD; idx += WARPS * 32) {
        const int h = idx / HD, d = idx % HD;
        const size_t base = (row + h0 + h) * n_chunks;
        float MM = NEG_BIG;
        for (int cc = c_lo; cc <= c_hi; ++cc)
            if (__ldcg(part_ml + (base + cc) * 2 + 1) > 0.f) MM = fmaxf(MM, __ldcg(part_ml + (base + cc) * 2));
        float L = 0.f, A = 0.f;
        for (int cc = c_lo; cc <= c_hi; ++cc) {
            const float lc = __ldcg(part_ml + (base + cc) * 2 + 1);
            if (lc > 0.f) {
                const float w = expf(__ldcg(part_ml + (base + cc) * 2) - MM);
                L = fmaf(w, lc, L);
                A = fmaf(w, __ldcg(part_acc + (base + cc) * HD + d), A);
            }
        }
        out[(size_t)t * o_stride + (size_t)(h0 + h) * HD + d] = __float2bfloat16_rn(L > 0.f ? A / L : 0.f);
    }
}

template <int HD, int GC>
int launch(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int* block_table,
           int max_pages, const int* seq_slot, const int* cu_q, const int* kv_len, int B, int nq, int nkv,
           float scale, int window, int n_chunks, float* part_acc, float* part_ml, int* counters, void* out,
           int o_stride, cudaStream_t s) {
    const int g = nq / nkv;
    dim3 grid(n_chunks, nkv * (g / GC), B);
    if (grid.y > 65535 || grid.z > 65535) return RB_ERR_BAD_SIZE;
    RB_LAUNCH((attention_decode_kernel<HD, GC>), dim3(grid), dim3(WARPS * 32), 0, s, 
        (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
        block_table, max_pages, seq_slot, cu_q, kv_len, nq, nkv, scale, window, n_chunks, part_acc, part_ml,
        counters, (__nv_bfloat16*)out, o_stride);
    RB_LAUNCH_CHECK();
    return RB_OK;
}
}  // namespace

// One query token per sequence (token index cu_q[b]).  chunk is fixed at 128 keys; n_chunks covers
// the longest sequence of the batch; with n_chunks == 1 the result is written to `out` directly.
// Work space: part_acc [T, nq, n_chunks, hd], part_ml [T, nq, n_chunks, 2] and `counters`, at least
// B * nkv * (group / heads per block) ints that are ZERO on entry and are left zero on exit.
// Returns RB_ERR_BAD_SIZE for head sizes other than 64, 128, 256 (the caller uses the plain kernel).
extern "C" int rb_attention_decode(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                   const int* block_table, int max_pages, const int* seq_slot, const int* cu_q,
                                   const int* kv_len, int B, int nq, int nkv, int hd, float scale, int window,
                                   int n_chunks, float* part_acc, float* part_ml, int* counters, void* out,
                                   int o_stride, void* stream) {
    if (B <= 0) return RB_OK;
    if (nkv <= 0 || nq % nkv || n_chunks < 1) return RB_ERR_BAD_SIZE;
    if (n_chunks > 1 && (!part_acc || !part_ml || !counters)) return RB_ERR_BAD_SIZE;
    if (((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15) || (q_stride % 8))
        return RB_ERR_BAD_ALIGN;
    cudaStream_t s = (cudaStream_t)stream;
    const int g = nq / nkv;
    const int gc = g % 4 == 0 ? 4 : (g % 2 == 0 ? 2 : 1);
#define RB_AD(HD, GC) return launch<HD, GC>(q, q_stride, k_cache, v_cache, block_table, max_pages, seq_slot, cu_q, \
                                            kv_len, B, nq, nkv, scale, window, n_chunks, part_acc, part_ml, counters, out, o_stride, s)
    if (hd == 128) { if (gc == 4) RB_AD(128, 4); if (gc == 2) RB_AD(128, 2); RB_AD(128, 1); }
    if (hd == 64) { if (gc == 4) RB_AD(64, 4); if (gc == 2) RB_AD(64, 2); RB_AD(64, 1); }
    if (hd == 256) { if (gc == 4) RB_AD(256, 2); if (gc == 2) RB_AD(256, 2); RB_AD(256, 1); }
#undef RB_AD
    return RB_ERR_BAD_SIZE;
}
