// Flash attention for bfloat16 prompts (and pieces of prompts) over the paged cache, on the tensor
// cores (mma.sync m16n8k16, float32 accumulation).
//
// A block takes 64 query tokens of one sequence and one query head; its 4 warps own 16 rows each.
// Keys and values are visited page by page (a page of the cache is exactly one 64-key tile, 16 KB
// contiguous at a head size of 128), double-buffered in shared memory with cp.async.  Shared-memory
// rows are stored with their 16-byte chunks XOR-swizzled by the row number so that ldmatrix reads
// are free of bank conflicts.  Per tile: S = Q K^T, scale, mask (causal, inclusive; window; end of
// the sequence), online softmax in float32, P (rounded to bfloat16) times V.  The query's position
// is its absolute position in its sequence, so a piece of a prompt attends to the cache that
// earlier steps left.
//
// Same mathematics as the reference's attn_prefill_* and attn_prefill_flash_* kernels
// (rocml-kernels/kernels/attn_prefill.hip:96-226, attn_prefill_flash_impl.h:46-159): head h reads
// key/value head h / g, score = (q.k) * scale, query at position p sees keys 0..p, softmax with the
// running maximum subtracted, o = sum p v / l.  Head sizes 64, 128, 256; others use the plain kernel.
#include "common.cuh"
#include "mma_tiles.cuh"
#include "api.h"

using namespace rb;
using namespace mma_tiles;

namespace {
constexpr int BM = 64;    // query rows per block
constexpr int BN = 64;    // keys per tile = one page
constexpr int NWARPS = 4;
constexpr float NEG_BIG = -1e30f;
constexpr float LOG2E = 1.4426950408889634f;

template <int HD>
__global__ void __launch_bounds__(NWARPS * 32)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out,
                         int o_stride, const __nv_bfloat16* __restrict__ k_cache,
                         const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_table,
                         int max_pages, const int* __restrict__ seq_slot, const int* __restrict__ cu_q,
                         const int* __restrict__ kv_len, int nq, int nkv, float scale, int window) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* Ks = Qs + BM * HD;          // [2][BN][HD]
    __nv_bfloat16* Vs = Ks + 2 * BN * HD;      // [2][BN][HD]

    const int b = blockIdx.z, head = blockIdx.y;
    const int slot = seq_slot[b];
    if (slot < 0) return;
    const int q0 = cu_q[b], q_len = cu_q[b + 1] - q0;
    const int m0 = blockIdx.x * BM;
    if (m0 >= q_len) return;
    const int len = kv_len[b];
    const int pos0 = len - q_len;                       // position of the sequence's first query token
    const int kvh = head / (nq / nkv);
    const int rows_here = min(BM, q_len - m0);
    const int hi = pos0 + m0 + rows_here - 1;           // last key any row of the block may see
    const int lo = window > 0 ? max(0, pos0 + m0 - window + 1) : 0;
    const int kt_first = lo / BN, kt_last = hi / BN;
    const int* table = block_table + (size_t)slot * max_pages;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;

    auto load_kv = [&](int kt, int buf) {
        const int page = table[kt];
        const size_t off = ((size_t)(page < 0 ? 0 : page) * nkv + kvh) * RB_PAGE * HD;
        const int valid = page < 0 ? 0 : min(BN, len - kt * BN);
        load_tile<HD>(Ks + buf * BN * HD, k_cache + off, HD, BN, valid, threadIdx.x, NWARPS * 32);
        load_tile<HD>(Vs + buf * BN * HD, v_cache + off, HD, BN, valid, threadIdx.x, NWARPS * 32);
    };

    load_tile<HD>(Qs, q + (size_t)(q0 + m0) * q_stride + (size_t)head * HD, q_stride, BM, rows_here, threadIdx.x,
                  NWARPS * 32);
    load_kv(kt_first, 0);
    cp_async_commit();

    // this warp's rows: m0 + warp*16 + g and + 8
    uint32_t qa[HD / 16][4];
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_run[2] = {NEG_BIG, NEG_BIG}, l_run[2] = {0.f, 0.f};
    const int row_pos[2] = {pos0 + m0 + warp * 16 + g, pos0 + m0 + warp * 16 + g + 8};
    const float sl2 = scale * LOG2E;
    const uint32_t qs_base = smem_addr(Qs);

    for (int kt = kt_first; kt <= kt_last; ++kt) {
        const int buf = (kt - kt_first) & 1;
        cp_async_wait<0>();
        __syncthreads();                                  // tile kt has landed; the other buffer is free
        if (kt + 1 <= kt_last) load_kv(kt + 1, buf ^ 1);
        cp_async_commit();
        if (kt == kt_first) {
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
                const int row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                ldmatrix_x4(tile_addr<HD>(qs_base, row, ks * 2 + (lane >> 4)), qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3]);
            }
        }
        const uint32_t ks_base = smem_addr(Ks + buf * BN * HD);
        const uint32_t vs_base = smem_addr(Vs + buf * BN * HD);

        // S = Q K^T: 16 rows x 64 keys per warp
        float s[BN / 8][4];
#pragma unroll
        for (int j = 0; j < BN / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
        for (int ks = 0; ks < HD / 16; ks += 2) {
#pragma unroll
            for (int j = 0; j < BN / 8; ++j) {
                uint32_t b0, b1, b2, b3;   // keys 8j..8j+7; dims 16ks..+15 (b0,b1) and 16(ks+1)..+15 (b2,b3)
                ldmatrix_x4(tile_addr<HD>(ks_base, j * 8 + (lane & 7), ks * 2 + (lane >> 3)), b0, b1, b2, b3);
                mma_bf16(s[j], qa[ks], b0, b1);
                mma_bf16(s[j], qa[ks + 1], b2, b3);
            }
        }
        // scale, mask, online softmax (base 2: exp(x) = exp2(x * log2 e))
        float mx[2] = {NEG_BIG, NEG_BIG};
#pragma unroll
        for (int j = 0; j < BN / 8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = kt * BN + j * 8 + t * 2 + (e & 1);
                const int r = e >> 1;
                const bool ok = key <= row_pos[r] && (window <= 0 || key > row_pos[r] - window);
                s[j][e] = ok ? s[j][e] * sl2 : -INFINITY;
                mx[r] = fmaxf(mx[r], s[j][e]);
            }
        }
        float alpha[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r]);
            alpha[r] = exp2f(m_run[r] - m_new);
            m_run[r] = m_new;
            l_run[r] *= alpha[r];
        }
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
            o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
            o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
        }
        uint32_t pa[BN / 16][4];
#pragma unroll
        for (int j = 0; j < BN / 8; ++j) {
            const float p0 = exp2f(s[j][0] - m_run[0]), p1 = exp2f(s[j][1] - m_run[0]);
            const float p2 = exp2f(s[j][2] - m_run[1]), p3 = exp2f(s[j][3] - m_run[1]);
            l_run[0] += p0 + p1;
            l_run[1] += p2 + p3;
            pa[j >> 1][(j & 1) * 2] = pack_bf16(p0, p1);
            pa[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
        // O += P V
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
#pragma unroll
            for (int i = 0; i < HD / 8; i += 2) {
                uint32_t b0, b1, b2, b3;   // keys 16kk..+15; dims 8i..8i+7 (b0,b1) and 8(i+1)..+7 (b2,b3)
                const int row = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                ldmatrix_x4_trans(tile_addr<HD>(vs_base, row, i + (lane >> 4)), b0, b1, b2, b3);
                mma_bf16(o[i], pa[kk], b0, b1);
                mma_bf16(o[i + 1], pa[kk], b2, b3);
            }
        }
    }
    cp_async_wait<0>();

    // normalise and store
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    const float inv0 = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f;
    const float inv1 = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
    const int r0 = m0 + warp * 16 + g, r1 = r0 + 8;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
        const int d = i * 8 + t * 2;
        if (r0 < q_len)
            *reinterpret_cast<uint32_t*>(out + (size_t)(q0 + r0) * o_stride + (size_t)head * HD + d) =
                pack_bf16(o[i][0] * inv0, o[i][1] * inv0);
        if (r1 < q_len)
            *reinterpret_cast<uint32_t*>(out + (size_t)(q0 + r1) * o_stride + (size_t)head * HD + d) =
                pack_bf16(o[i][2] * inv1, o[i][3] * inv1);
    }
}

template <int HD>
int launch(const void* q, int q_stride, void* out, int o_stride, const void* k_cache, const void* v_cache,
           const int* block_table, int max_pages, const int* seq_slot, const int* cu_q, const int* kv_len, int B,
           int max_q_len, int nq, int nkv, float scale, int window, cudaStream_t s) {
    const size_t smem = (size_t)(BM + 4 * BN) * HD * sizeof(__nv_bfloat16);
    auto k = attention_prefill_kernel<HD>;
    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        attr_done = true;
    }
    dim3 grid((max_q_len + BM - 1) / BM, nq, B);
    if (grid.y > 65535 || grid.z > 65535) return RB_ERR_BAD_SIZE;
    RB_LAUNCH((k), grid, dim3(NWARPS * 32), smem, s, (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out,
              o_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, block_table, max_pages,
              seq_slot, cu_q, kv_len, nq, nkv, scale, window);
    return RB_OK;
}
}  // namespace

// q rows [T, >= nq*hd] bfloat16 -> out rows; keys and values from the pages.  Returns
// RB_ERR_BAD_SIZE for head sizes other than 64, 128, 256 and RB_ERR_BAD_ALIGN for rows or pointers
// off a 16-byte boundary (the caller then uses the plain kernel).
extern "C" int rb_attention_prefill(const void* q, int q_stride, void* out, int o_stride, const void* k_cache,
                                    const void* v_cache, const int* block_table, int max_pages,
                                    const int* seq_slot, const int* cu_q, const int* kv_len, int B, int max_q_len,
                                    int nq, int nkv, int hd, float scale, int window, void* stream) {
    if (B <= 0 || max_q_len <= 0) return RB_OK;
    if (nkv <= 0 || nq % nkv) return RB_ERR_BAD_SIZE;
    if (((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15) || ((uintptr_t)out & 3) ||
        (q_stride % 8) || (o_stride % 2))
        return RB_ERR_BAD_ALIGN;
    cudaStream_t s = (cudaStream_t)stream;
#define RB_AP(HD) return launch<HD>(q, q_stride, out, o_stride, k_cache, v_cache, block_table, max_pages, seq_slot, \
                                    cu_q, kv_len, B, max_q_len, nq, nkv, scale, window, s)
    if (hd == 128) RB_AP(128);
    if (hd == 64) RB_AP(64);
    if (hd == 256) RB_AP(256);
#undef RB_AP
    return RB_ERR_BAD_SIZE;
}
