// Plain attention over the paged cache on the CUDA cores, 32-bit arithmetic, any element type.
//
// One kernel serves whole prompts, chunks of prompts that continue a cache, and single
// decoded tokens: every query row (token, head) attends to the keys of its own sequence at
// positions lo..pos with pos the token's absolute position (causal, inclusive:
// rocml-kernels/kernels/attn_prefill.hip:57-60,121) and lo = max(0, pos - window + 1) when the
// layer has a window.  Query head h reads key/value head h / g (attn_decode.hip:108); the
// score is (q . k) * scale, scale applied after the dot (attn_decode.hip:158); softmax is an
// online max/sum in 32-bit with expf (attn_decode.hip:160-170); o = sum p v / l
// (attn_prefill.hip:201-203).
//
// Keys are visited in tiles of 32 aligned to absolute positions, so the order of every row's
// sums depends on its own position only, never on the batch or on how the prompt was cut.
// With `chunk` > 0 the keys are split in fixed chunks of that many positions (again from
// position 0, independent of the batch); each chunk writes an unnormalised partial result and
// rb_attention_merge combines them in ascending order (the reference's split-K pair
// attn_decode_partial_* + attn_decode_reduce_f32, attn_decode.hip:93-255).
//
// This kernel is the attention of the true 32-bit path and the reference the tensor-core
// kernels are tested against.
#include <type_traits>
#include "common.cuh"
#include "api.h"
#include <math.h>

using namespace rb;

namespace {
constexpr int ROWS = 16;       // query rows (token, head) per block
constexpr int RW = 4;          // rows per warp
constexpr int KT = 32;         // keys per tile: one per lane
constexpr int MAX_DPL = 8;     // head dims per lane -> head size up to 256
constexpr float NEG_BIG = -1e30f;

__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}

template <typename T>
__global__ void __launch_bounds__(128, 4)
attention_generic_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int o_stride,
                         const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                         const int* __restrict__ block_table, int max_pages,
                         const int* __restrict__ seq_slot, const int* __restrict__ cu_q,
                         const int* __restrict__ kv_len, int nq, int nkv, int hd, float scale, int window,
                         int chunk, int n_chunks, float* __restrict__ part_acc,
                         float* __restrict__ part_ml) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    const int g = nq / nkv;
    const int HG = g < ROWS ? g : ROWS;           // heads of the group handled by this block
    const int QB = ROWS / HG;                     // query tokens per block
    const int head_chunks = (g + HG - 1) / HG;
    const int b = blockIdx.z;
    const int kvh = blockIdx.y / head_chunks;
    const int hc = blockIdx.y % head_chunks;
    const int qblk = blockIdx.x / n_chunks;
    const int c = blockIdx.x % n_chunks;

    const int slot = seq_slot[b];
    if (slot < 0) return;
    const int q0 = cu_q[b], q_len = cu_q[b + 1] - q0;
    const int tok0 = qblk * QB;
    if (tok0 >= q_len) return;
    const int len = kv_len[b];
    const int pos0 = len - q_len;  // absolute position of the sequence's first query token
    // a chunk that lies wholly after this block's last query has nothing to do and is never merged
    if (chunk > 0 && c * chunk > pos0 + min(tok0 + QB, q_len) - 1) return;

    float* q_s = smem;                               // [ROWS][hd]
    float* k_s = q_s + ROWS * hd;                    // [KT][hd + 1]
    float* v_s = k_s + KT * (hd + 1);                // [KT][hd]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // rows of this block: r -> (token tok0 + r / HG, head kvh*g + hc*HG + r % HG)
    if ((hd & 3) == 0 && (q_stride & 3) == 0 && ((uintptr_t)q & (4 * sizeof(T) - 1)) == 0) {
        // four elements a load; the loads of a thread's rows do not wait for one another
        const int hd4 = hd >> 2;
        for (int i0 = tid; i0 < ROWS * hd4; i0 += blockDim.x * 4) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i4 = i0 + u * blockDim.x;
                const int r = i4 / hd4, d4 = i4 - r * hd4;
                const int qi = tok0 + r / HG, hg = hc * HG + r % HG;
                v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (i4 < ROWS * hd4 && r < QB * HG && qi < q_len && hg < g)
                    v[u] = load4(q + (size_t)(q0 + qi) * q_stride + (size_t)(kvh * g + hg) * hd + d4 * 4);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i4 = i0 + u * blockDim.x;
                if (i4 < ROWS * hd4) *reinterpret_cast<float4*>(q_s + i4 * 4) = v[u];
            }
        }
    } else {
        for (int idx = tid; idx < ROWS * hd; idx += blockDim.x) {
            const int r = idx / hd, d = idx - r * hd;
            const int qi = tok0 + r / HG, hg = hc * HG + r % HG;
            float v = 0.f;
            if (r < QB * HG && qi < q_len && hg < g)
                v = to_f32(q[(size_t)(q0 + qi) * q_stride + (size_t)(kvh * g + hg) * hd + d]);
            q_s[idx] = v;
        }
    }

    int row_pos[RW], row_lo[RW];
    bool row_ok[RW];
    float m[RW], l[RW], acc[RW][MAX_DPL];
#pragma unroll
    for (int i = 0; i < RW; ++i) {
        const int r = i * 4 + warp;               // the block's rows are dealt out over its four warps in turn
        const int qi = tok0 + r / HG, hg = hc * HG + r % HG;
        row_ok[i] = r < QB * HG && qi < q_len && hg < g;
        row_pos[i] = pos0 + qi;
        row_lo[i] = window > 0 ? max(0, row_pos[i] - window + 1) : 0;
        m[i] = NEG_BIG;
        l[i] = 0.f;
#pragma unroll
        for (int j = 0; j < MAX_DPL; ++j) acc[i][j] = 0.f;
    }

    // A block with few rows (a decode step: one token, the group's heads) gives each warp one of them instead of
    // all to the first warp, and a warp works on the rows it has: n_rows of them if they are its first ones
    // (the usual case), all four otherwise.
    int n_rows = 0;
    {
        bool prefix = true;
#pragma unroll
        for (int i = 0; i < RW; ++i) {
            if (row_ok[i]) { if (n_rows != i) prefix = false; ++n_rows; }
        }
        if (!prefix) n_rows = RW;
    }

    // key range of the whole block, then of this chunk
    const int last_tok = min(tok0 + QB, q_len) - 1;
    int hi = pos0 + last_tok;                                       // inclusive
    int lo = window > 0 ? max(0, pos0 + tok0 - window + 1) : 0;
    if (chunk > 0) {
        lo = max(lo, c * chunk);
        hi = min(hi, (c + 1) * chunk - 1);
    }
    const int* table = block_table + (size_t)slot * max_pages;
    // four elements a load where the head size and the caches' addresses allow (pages, heads and keys then all
    // start on a multiple of four elements); blockDim.x is 128 (launch_attn)
    const bool vec = (hd & 3) == 0 && (((uintptr_t)k_cache | (uintptr_t)v_cache) & (4 * sizeof(T) - 1)) == 0 &&
                     ((ROWS * hd + KT * (hd + 1)) & 3) == 0;

    for (int t0 = (lo / KT) * KT; t0 <= hi; t0 += KT) {
        __syncthreads();  // previous tile fully consumed (and q_s written, first time)
        const int page = table[t0 / RB_PAGE];
        const size_t base = page >= 0 ? (((size_t)page * nkv + kvh) * RB_PAGE + (t0 % RB_PAGE)) * hd : 0;
        if (vec) {
            // A warp takes every fourth key, a lane four consecutive dimensions at a time, and all of a thread's
            // loads are requested before the first is stored: taken one element at a time, each load waited
            // for the one before, and a tile took as long as sixty-four trips to memory.
            constexpr int KPW = KT / 4;                           // keys per warp (4 warps a block)
            for (int d4 = lane; d4 < (hd >> 2); d4 += 32) {
                float4 kk[KPW], vv[KPW];
#pragma unroll
                for (int u = 0; u < KPW; ++u) {
                    const int jj = warp + 4 * u;
                    const bool in = page >= 0 && t0 + jj <= hi && t0 + jj >= lo;
                    const size_t off = base + (size_t)jj * hd + d4 * 4;
                    kk[u] = in ? load4(k_cache + off) : make_float4(0.f, 0.f, 0.f, 0.f);
                    vv[u] = in ? load4(v_cache + off) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int u = 0; u < KPW; ++u) {
                    const int jj = warp + 4 * u;
                    float* kd = k_s + jj * (hd + 1) + d4 * 4;
                    kd[0] = kk[u].x; kd[1] = kk[u].y; kd[2] = kk[u].z; kd[3] = kk[u].w;
                    *reinterpret_cast<float4*>(v_s + jj * hd + d4 * 4) = vv[u];
                }
            }
        } else {
            for (int idx = tid; idx < KT * hd; idx += blockDim.x) {
                const int jj = idx / hd, d = idx - jj * hd;
                const bool in = page >= 0 && t0 + jj <= hi && t0 + jj >= lo;
                k_s[jj * (hd + 1) + d] = in ? to_f32(k_cache[base + idx]) : 0.f;
                v_s[idx] = in ? to_f32(v_cache[base + idx]) : 0.f;
            }
        }
        __syncthreads();

        const int j = t0 + lane;
        auto work = [&](auto nr) {
            constexpr int NR = decltype(nr)::value;
            float s[NR];
#pragma unroll
            for (int i = 0; i < NR; ++i) s[i] = 0.f;
            const float* kr = k_s + lane * (hd + 1);
            for (int d = 0; d < hd; ++d) {
                const float kv = kr[d];
#pragma unroll
                for (int i = 0; i < NR; ++i) s[i] = fmaf(q_s[(i * 4 + warp) * hd + d], kv, s[i]);
            }
            float p[NR];
#pragma unroll
            for (int i = 0; i < NR; ++i) {
                const bool valid = row_ok[i] && j <= row_pos[i] && j >= row_lo[i] && j <= hi && j >= lo;
                const float sv = s[i] * scale;
                const float tmax = warp_max(valid ? sv : NEG_BIG);
                const float m_new = fmaxf(m[i], tmax);
                const float alpha = expf(m[i] - m_new);
                p[i] = valid ? expf(sv - m_new) : 0.f;
                l[i] = l[i] * alpha + warp_sum(p[i]);
                m[i] = m_new;
#pragma unroll
                for (int dd = 0; dd < MAX_DPL; ++dd) acc[i][dd] *= alpha;
            }
            for (int jj = 0; jj < KT; ++jj) {
                float pj[NR];
#pragma unroll
                for (int i = 0; i < NR; ++i) pj[i] = __shfl_sync(0xffffffffu, p[i], jj);
#pragma unroll
                for (int dd = 0; dd < MAX_DPL; ++dd) {
                    const int d = lane + 32 * dd;
                    if (d < hd) {
                        const float vv = v_s[jj * hd + d];
#pragma unroll
                        for (int i = 0; i < NR; ++i) acc[i][dd] = fmaf(pj[i], vv, acc[i][dd]);
                    }
                }
            }
        };
        if (n_rows == RW) work(std::integral_constant<int, RW>());
        else if (n_rows == 1) work(std::integral_constant<int, 1>());
        else if (n_rows == 2) work(std::integral_constant<int, 2>());
        else if (n_rows == 3) work(std::integral_constant<int, 3>());
    }

#pragma unroll
    for (int i = 0; i < RW; ++i) {
        if (!row_ok[i]) continue;
        const int r = i * 4 + warp;
        const int t = q0 + tok0 + r / HG;
        const int head = kvh * g + hc * HG + r % HG;
        if (chunk > 0) {
            const size_t pidx = ((size_t)t * nq + head) * n_chunks + c;
            if (lane == 0) { part_ml[pidx * 2] = m[i]; part_ml[pidx * 2 + 1] = l[i]; }
#pragma unroll
            for (int dd = 0; dd < MAX_DPL; ++dd) {
                const int d = lane + 32 * dd;
                if (d < hd) part_acc[pidx * hd + d] = acc[i][dd];
            }
        } else {
            const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
#pragma unroll
            for (int dd = 0; dd < MAX_DPL; ++dd) {
                const int d = lane + 32 * dd;
                if (d < hd) out[(size_t)t * o_stride + (size_t)head * hd + d] = from_f32<T>(acc[i][dd] * inv);
            }
        }
    }
}

// Combine the chunks' partial results of every (token, head), in ascending chunk order.
// One warp per (token, head): the lanes first walk the chunks for the maximum and the weights
// exp(m_c - M) (kept in shared memory), then each lane sums its head dimensions over the chunks.
template <typename T>
__global__ void attention_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                       T* __restrict__ out, int o_stride, const int* __restrict__ positions,
                                       const int* __restrict__ slot_of_token, int T_tokens, int nq, int hd,
                                       int chunk, int n_chunks, int window) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float w_s[];   // [warps][n_chunks]
    const int warps = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * warps + warp;
    if (item >= (long long)T_tokens * nq) return;
    const int t = (int)(item / nq), head = (int)(item % nq);
    if (slot_of_token[t] < 0) return;
    const int pos = positions[t];
    const int c_hi = min(n_chunks - 1, pos / chunk);
    const int c_lo = window > 0 ? max(0, pos - window + 1) / chunk : 0;
    const size_t base = ((size_t)t * nq + head) * n_chunks;
    float* w = w_s + (size_t)warp * n_chunks;
    float M = NEG_BIG;
    for (int c = c_lo + lane; c <= c_hi; c += 32)
        if (part_ml[(base + c) * 2 + 1] > 0.f) M = fmaxf(M, part_ml[(base + c) * 2]);
    M = warp_max(M);
    float L = 0.f;
    for (int c = c_lo + lane; c <= c_hi; c += 32) {
        const float lc = part_ml[(base + c) * 2 + 1];
        const float wc = lc > 0.f ? expf(part_ml[(base + c) * 2] - M) : 0.f;
        w[c] = wc;
        L += wc * lc;
    }
    L = warp_sum(L);
    __syncwarp();
    const float inv = L > 0.f ? 1.f / L : 0.f;
    for (int d = lane; d < hd; d += 32) {
        float a = 0.f;
        for (int c0 = c_lo; c0 <= c_hi; c0 += 8) {        // eight chunks' values in flight, added in ascending order
            float pa[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) pa[j] = c0 + j <= c_hi ? part_acc[(base + c0 + j) * hd + d] : 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (c0 + j <= c_hi) a = fmaf(w[c0 + j], pa[j], a);
        }
        out[(size_t)t * o_stride + (size_t)head * hd + d] = from_f32<T>(a * inv);
    }
}

template <typename T>
int launch_attn(const void* q, int q_stride, void* out, int o_stride, const void* k_cache, const void* v_cache,
                const int* block_table, int max_pages, const int* seq_slot, const int* cu_q,
                const int* kv_len, int B, int max_q_len, int nq, int nkv, int hd, float scale, int window,
                int chunk, int n_chunks, float* part_acc, float* part_ml, cudaStream_t s) {
    const int g = nq / nkv;
    const int HG = g < ROWS ? g : ROWS;
    const int QB = ROWS / HG;
    const int head_chunks = (g + HG - 1) / HG;
    const long long gx = (long long)((max_q_len + QB - 1) / QB) * n_chunks;
    if (gx > 0x7fffffffLL || (long long)nkv * head_chunks > 65535 || B > 65535) return RB_ERR_BAD_SIZE;
    const size_t smem = (size_t)(ROWS * hd + KT * (hd + 1) + KT * hd) * sizeof(float);
    auto k = attention_generic_kernel<T>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    dim3 grid((unsigned)gx, nkv * head_chunks, B);
    RB_LAUNCH((k), dim3(grid), dim3(128), smem, s, (const T*)q, q_stride, (T*)out, o_stride, (const T*)k_cache, (const T*)v_cache,
                              block_table, max_pages, seq_slot, cu_q, kv_len, nq, nkv, hd, scale, window,
                              chunk, n_chunks, part_acc, part_ml);
    RB_LAUNCH_CHECK();
    return RB_OK;
}
}  // namespace

extern "C" int rb_attention_generic(const void* q, int q_stride, void* out, int o_stride, int dtype,
                                    const void* k_cache, const void* v_cache, const int* block_table,
                                    int max_pages, const int* seq_slot, const int* cu_q, const int* kv_len,
                                    int B, int max_q_len, int nq, int nkv, int hd, float scale, int window,
                                    int chunk, int n_chunks, float* part_acc, float* part_ml, void* stream) {
    if (B <= 0 || max_q_len <= 0) return RB_OK;
    if (hd <= 0 || hd > 32 * MAX_DPL || nkv <= 0 || nq % nkv) return RB_ERR_BAD_SIZE;
    if (chunk > 0 && (chunk % KT || n_chunks <= 0 || !part_acc || !part_ml)) return RB_ERR_BAD_SIZE;
    if (chunk <= 0) n_chunks = 1;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RB_BF16)
        return launch_attn<__nv_bfloat16>(q, q_stride, out, o_stride, k_cache, v_cache, block_table, max_pages,
                                          seq_slot, cu_q, kv_len, B, max_q_len, nq, nkv, hd, scale, window,
                                          chunk, n_chunks, part_acc, part_ml, s);
    if (dtype == RB_F32)
        return launch_attn<float>(q, q_stride, out, o_stride, k_cache, v_cache, block_table, max_pages, seq_slot,
                                  cu_q, kv_len, B, max_q_len, nq, nkv, hd, scale, window, chunk, n_chunks,
                                  part_acc, part_ml, s);
    return RB_ERR_BAD_DTYPE;
}

extern "C" int rb_attention_merge(const float* part_acc, const float* part_ml, void* out, int o_stride,
                                  int dtype, const int* positions, const int* slot_of_token, int T, int nq,
                                  int hd, int chunk, int n_chunks, int window, void* stream) {
    if (T <= 0) return RB_OK;
    if (chunk <= 0 || n_chunks <= 0) return RB_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const int warps = 4;
    const long long blocks = ((long long)T * nq + warps - 1) / warps;
    if (blocks > 0x7fffffffLL) return RB_ERR_BAD_SIZE;
    const size_t smem = (size_t)warps * n_chunks * sizeof(float);
    if (smem > 48 * 1024) return RB_ERR_BAD_SIZE;
    if (dtype == RB_BF16)
        RB_LAUNCH((attention_merge_kernel<__nv_bfloat16>), dim3((int)blocks), dim3(warps * 32), smem, s, part_acc, part_ml, (__nv_bfloat16*)out, o_stride,
                                                                  positions, slot_of_token, T, nq, hd, chunk,
                                                                  n_chunks, window);
    else if (dtype == RB_F32)
        RB_LAUNCH((attention_merge_kernel<float>), dim3((int)blocks), dim3(warps * 32), smem, s, part_acc, part_ml, (float*)out, o_stride,
                                                                  positions, slot_of_token, T, nq, hd, chunk,
                                                                  n_chunks, window);
    else
        return RB_ERR_BAD_DTYPE;
    RB_LAUNCH_CHECK();
    return RB_OK;
}
