// Decode attention over the paged cache for bfloat16: one query token per sequence, keys split in
// fixed chunks of 64, one page each (split-KV), the chunks' partial results merged by the block that finishes last.
//
// The kernel is bound by reading the cache once.  A block takes one (chunk, key/value head, sequence)
// and all query heads of the group (up to 16), which share every key and value it reads: the heads
// are the rows of a 16-row tensor-core tile (mma.sync m16n8k16, float32 accumulation), so the
// arithmetic costs next to nothing whatever the group size.  Each of the 4 warps copies its own 16
// keys and 16 values into shared memory with cp.async (16-byte chunks, XOR-swizzled for ldmatrix),
// computes S = Q K^T, the softmax statistics of its keys and P V, and the warps' results are merged
// through shared memory.  Then the blocks of one (sequence, head group) merge their partial results,
// in ascending order of the keys.  Up to 16 of them are launched as one thread-block cluster: each
// keeps its part in its own shared memory, and after a cluster barrier each merges one slice of the
// head size, reading the others' parts through distributed shared memory.  More blocks than that
// write unnormalised partial results to global memory; a counter per (sequence, head group) tells
// the last block to arrive, which merges all chunks and writes the output (the counter is left at
// zero for the next launch).  Softmax is float32, base 2 (exp(x) = exp2(x log2 e)).
//
// Replaces attn_decode_partial_f16 + attn_decode_reduce_f32 of the reference
// (rocml-kernels/kernels/attn_decode.hip:93-255): same mathematics (head h reads key/value head
// h / g, score = (q.k) * scale, max/sum softmax, split over the keys, log-sum-exp merge), other
// mapping.  Head sizes 64, 128 and 256; other sizes use the plain kernel.
#include "common.cuh"
#include "mma_tiles.cuh"
#include "api.h"
#include <cstdlib>

using namespace rb;
using namespace mma_tiles;

namespace {
constexpr int CHUNK = 64;         // keys per block: one page
constexpr int WARPS = 4;
constexpr int WK = CHUNK / WARPS; // keys per warp: 16
constexpr int ROWS = 16;          // query heads per block (rows of the MMA tile)
constexpr int MAX_CLUSTER = 16;   // blocks of one (sequence, head group) that can form a cluster (8 is the portable size)
constexpr float NEG_BIG = -1e30f;
constexpr float LOG2E = 1.4426950408889634f;

// 2^x on the special-function unit, one instruction (x <= 0 here, -inf gives 0); the library's exp2f
// adds range handling that the softmax does not need.
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Blocks of one (sequence, head group) as one thread-block cluster (CL): see the merge below.
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_cluster(const float* local, unsigned rank) {
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_addr(local)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

// FQ (head size 128): the step's projections arrive as they leave the matrix product (float32 partial
// sums over K, [S][T][q heads | k heads | v heads]) and the kernel does what a kernel of its own would
// otherwise do between the two: it adds the partial sums, normalises each query head (RMSNorm over the
// head, float32), rotates it (NEOX pairs i, i + 64; cos/sin from the step's table) and keeps it in
// shared memory; the one block that reads the page of the new token does the same for that token's key,
// and writes key and value into the page before it copies the page.
struct Projections {
    const float* proj;        // null: queries are read from `q`, the cache is already written
    int n_in;                 // partial sums
    long long in_stride;      // elements between two partial sums
    int row_stride;           // elements between two tokens
    const void* q_norm_w;     // [128] or null (no norm)
    const void* k_norm_w;
    int w_f32;                // the norm weights' type: float32 or bfloat16
    float eps;
    const float2* cos_sin;    // [T][64] (cos, sin) or null (no rotation)
    int write_kv;             // 0: this layer reads a cache that another layer wrote
    __nv_bfloat16* k_out;     // the cache to write (k_cache / v_cache of the call)
    __nv_bfloat16* v_out;
    // The rows the projection was made from may still lack their norm's 1/RMS (they were residual *
    // weight): then the sums are scaled by it here, from shares of the rows' sums of squares.
    const float* row_sumsq;   // [row_groups][tokens], or null
    int row_groups;
    long long row_sumsq_ld;
    float row_eps, row_inv_width;
};

// One head of 128 values, 4 per lane: the sum of the partial sums, then (what != 2) RMSNorm with `w`
// and the rotation by the token's angles.  what: 0 query, 1 key, 2 value.
__device__ __forceinline__ void project_head(const Projections& pj, const float* src, int what, int t, int lane,
                                             float sumsq_share, float* v) {
    v[0] = v[1] = v[2] = v[3] = 0.f;
    // the norm's weights and the token's angles do not depend on the sums: their loads go out first
    const void* w = what == 0 ? pj.q_norm_w : (what == 1 ? pj.k_norm_w : nullptr);
    const bool rotate = what != 2 && pj.cos_sin != nullptr;
    float wj[4] = {1.f, 1.f, 1.f, 1.f};
    float2 cs[4];
    if (w != nullptr) {
        if (pj.w_f32) {
            const float4 f = *reinterpret_cast<const float4*>(static_cast<const float*>(w) + lane * 4);
            wj[0] = f.x; wj[1] = f.y; wj[2] = f.z; wj[3] = f.w;
        } else {
            const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(w) + lane * 4);
            const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
            const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
            wj[0] = a.x; wj[1] = a.y; wj[2] = b.x; wj[3] = b.y;
        }
    }
    if (rotate) {
        const float4* c4 = reinterpret_cast<const float4*>(pj.cos_sin + (size_t)t * 64 + (lane & 15) * 4);
        const float4 a = c4[0], b = c4[1];
        cs[0] = make_float2(a.x, a.y); cs[1] = make_float2(a.z, a.w);
        cs[2] = make_float2(b.x, b.y); cs[3] = make_float2(b.z, b.w);
    }
    for (int s = 0; s < pj.n_in; s += 8) {                  // eight partial sums in flight, added in order
        float4 f[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            f[j] = s + j < pj.n_in ? *reinterpret_cast<const float4*>(src + (size_t)(s + j) * pj.in_stride)
                                   : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 8; ++j) { v[0] += f[j].x; v[1] += f[j].y; v[2] += f[j].z; v[3] += f[j].w; }
    }
    // the rows' 1/RMS, if it is still to be applied: reduced here, after the loads above went out
    if (pj.row_sumsq != nullptr) {
        const float rstd = rsqrtf(warp_sum(sumsq_share) * pj.row_inv_width + pj.row_eps);
        v[0] *= rstd; v[1] *= rstd; v[2] *= rstd; v[3] *= rstd;
    }
    if (w != nullptr) {
        const float ss = warp_sum(v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3]);
        const float inv = rsqrtf(ss / 128.f + pj.eps);
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = v[j] * inv * wj[j];
    }
    if (rotate) {
        // dimension i < 64 pairs with i + 64: lanes 0-15 hold x_i, lanes 16-31 the partners
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float other = __shfl_xor_sync(0xffffffffu, v[j], 16);
            v[j] = lane < 16 ? v[j] * cs[j].x - other * cs[j].y : other * cs[j].y + v[j] * cs[j].x;
        }
    }
}
__device__ __forceinline__ uint2 pack4_bf16(const float* v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&lo);
    raw.y = *reinterpret_cast<uint32_t*>(&hi);
    return raw;
}

// PROP (long contexts of unequal lengths; more sequences than blocks fit the device at once): the grid's
// x blocks of a head group are not tied to one sequence each; the sequences' pages, laid end to end, are
// cut into equal runs, one per block, so that every block reads the same number of bytes whatever the
// lengths and the batch.  grid = (blocks, groups, 1).
constexpr int PROP_MAX_SEQS = 256;

// TR (groups of at most 8 query heads, which is every size of the architecture): the products are
// transposed.  S^T = K Q^T has the 16 keys of a warp's slice as the rows of the MMA tile and the heads as
// its 8 columns, and O^T = V^T P the head size as rows: half the MMAs, half the softmax arithmetic and
// half the accumulator registers of the layout with 16 head rows, of which a group of 4 fills a quarter.
// P leaves the first product with keys along the lanes' groups and enters the second with keys along a
// lane's pairs: one movmatrix per 8 keys transposes it in registers.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

template <int HD, bool CL, bool FQ, bool PROP, bool TR>
__global__ void __launch_bounds__(WARPS * 32, HD <= 128 ? 3 : 1)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, int q_stride,
                        const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                        const int* __restrict__ block_table, int max_pages, const int* __restrict__ seq_slot,
                        const int* __restrict__ cu_q, const int* __restrict__ kv_len, int nq, int nkv,
                        float scale, int window, int n_chunks, int ppb, float* __restrict__ part_acc,
                        float* __restrict__ part_ml, int* __restrict__ counters,
                        __nv_bfloat16* __restrict__ out, int o_stride, const Projections pj, int n_seqs) {
    pdl_trigger();
    // Everything up to pdl_wait() below may run while the kernels before this one in the stream are
    // still running.  It reads the step's integers (copied to the device before the step's first
    // kernel) and pages of keys and values that EARLIER steps wrote; the one page of a sequence that
    // receives this step's token, and the queries, are read after the wait.
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);        // [16][HD]
    __nv_bfloat16* KVs = Qs + ROWS * HD;                                    // per warp: K [32][HD], V [32][HD]
    float* s_o = reinterpret_cast<float*>(KVs);                            // reused after the products: [4][16][HD]
    float* s_part = s_o + WARPS * ROWS * HD;                               // beside it (CL): this block's part [16][HD]
    __shared__ float s_pm_own[ROWS], s_pl_own[ROWS];                       // its maxima and sums
    __shared__ float s_m[WARPS][ROWS], s_l[WARPS][ROWS];
    __shared__ int s_last;

    const int g = nq / nkv;
    const int head_chunks = (g + ROWS - 1) / ROWS;
    const int kvh = blockIdx.y / head_chunks;
    const int hc = blockIdx.y % head_chunks;
    const int h0 = kvh * g + hc * ROWS;                     // first query head of this block
    const int rows_valid = min(ROWS, g - hc * ROWS);
    int c = blockIdx.x, b = blockIdx.z;
    // PROP: the pages that the sequences of this head group visit, laid end to end, are cut into equal
    // runs, one per block of the grid's x; a run may end one sequence and begin the next, so a block works
    // in rounds, one per sequence that its run touches
    long long run_lo = 0, run_hi = 0, seq_start = 0, total = 0;
    int n_runs = 1, seq_next = 0;
    __shared__ int s_pages[PROP ? PROP_MAX_SEQS : 1];
    if (PROP) {
        for (int i = threadIdx.x; i < n_seqs; i += WARPS * 32) {
            const int ps = kv_len[i] - 1;
            int P = 0;
            if (seq_slot[i] >= 0 && ps >= 0) P = ps / CHUNK - (window > 0 ? max(0, ps - window + 1) / CHUNK : 0) + 1;
            s_pages[i] = P;
        }
        __syncthreads();
        for (int i = 0; i < n_seqs; ++i) total += s_pages[i];
        n_runs = (int)min((long long)gridDim.x, total);     // every run holds a page at least
        if ((int)blockIdx.x >= n_runs) return;
        run_lo = (long long)blockIdx.x * total / n_runs;
        run_hi = (long long)(blockIdx.x + 1) * total / n_runs;
    }
  for (;;) {
   {
    int page_first, page_last, parts_lo, parts_hi;         // this block's pages, and the parts that exist of this (sequence, group)
    if (PROP) {
        // the next sequence that the run touches
        while (seq_next < n_seqs && seq_start + s_pages[seq_next] <= run_lo) seq_start += s_pages[seq_next++];
        if (seq_next >= n_seqs || seq_start >= run_hi) return;
        b = seq_next;
    }
    const int slot = seq_slot[b];
    if (slot < 0) return;
    const int t = cu_q[b];
    const int pos = kv_len[b] - 1;
    const int win_lo = window > 0 ? max(0, pos - window + 1) : 0;
    // this block's pages: [c * ppb, (c + 1) * ppb), cut at the sequence's end; PROP: what the run holds
    // of the sequence's visited pages
    if (PROP) {
        const long long P = s_pages[b];
        const int first = win_lo / CHUNK;
        page_first = first + (int)(max(run_lo, seq_start) - seq_start);
        page_last = first + (int)(min(run_hi, seq_start + P) - seq_start) - 1;
        // the runs that hold the sequence's first and last page: its parts are numbered from the first
        const int x_first = (int)(((seq_start + 1) * n_runs + total - 1) / total) - 1;
        const int x_last = (int)(((seq_start + P) * n_runs + total - 1) / total) - 1;
        c = (int)blockIdx.x - x_first;
        parts_lo = 0;
        parts_hi = x_last - x_first;
        seq_start += P;                                     // the round after this one starts at the next sequence
        ++seq_next;
    } else {
        page_first = c * ppb;
        // beyond the sequence: takes no part in the merge; in a cluster it stays, with an empty result
        if (!CL && page_first * CHUNK > pos) return;
        page_last = min(pos / CHUNK, page_first + ppb - 1);
        parts_hi = pos / (CHUNK * ppb);
        parts_lo = win_lo / (CHUNK * ppb);
    }

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gq = lane >> 2, tq = lane & 3;
    const int* table = block_table + (size_t)slot * max_pages;

    // Each warp owns 16 keys of every page and two shared-memory buffers for them: while it
    // works on one page its copies of the next are in flight.
    __nv_bfloat16* KVw = KVs + warp * 4 * WK * HD;          // [2 buffers][K 16 x HD | V 16 x HD]
    auto issue = [&](int page_idx, int buf) {
        const int j0 = page_idx * CHUNK + warp * WK;
        const int hi = min(pos, (page_idx + 1) * CHUNK - 1);
        const bool any = page_idx <= page_last && j0 <= hi && j0 + WK - 1 >= win_lo;
        if (any) {
            const int page = table[page_idx];
            const size_t off = (((size_t)(page < 0 ? 0 : page) * nkv + kvh) * RB_PAGE + warp * WK) * HD;
            const int valid = page < 0 ? 0 : min(WK, hi - j0 + 1);   // rows past the sequence's end are zero-filled
            __nv_bfloat16* Kw = KVw + buf * 2 * WK * HD;
            load_tile<HD>(Kw, k_cache + off, HD, WK, valid, lane, 32);
            load_tile<HD>(Kw + WK * HD, v_cache + off, HD, WK, valid, lane, 32);
        }
        cp_async_commit();
    };
    // Two pages in flight per warp.  A page below the one that holds position `pos` was complete
    // before this step began, so its copies start at once; the others start after the wait.
    const int new_page = pos / CHUNK;
    const bool early0 = page_first < new_page, early1 = page_first + 1 < new_page;
    if (early0) issue(page_first, 0);
    if (early1) issue(page_first + 1, 1);
    pdl_wait();
    if (FQ) {
        const float* row = pj.proj + (size_t)t * pj.row_stride;
        float share = 0.f;                                  // this lane's share of the row's sum of squares
        if (pj.row_sumsq != nullptr) {
            for (int g0 = 0; g0 < pj.row_groups; g0 += 256) {   // eight loads a lane in flight, not one after another
                float x[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int gi = g0 + j * 32 + lane;
                    x[j] = gi < pj.row_groups ? pj.row_sumsq[(size_t)gi * pj.row_sumsq_ld + t] : 0.f;
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) share += x[j];
            }
        }
        // The new token's key and value first, by the one block that reads their page (its last two
        // warps), so that the page's copies are on their way while the query heads are made.
        const bool owner = pj.write_kv && hc == 0 && page_first <= new_page && new_page <= page_last;
        if (owner) {
            if (warp >= WARPS - 2) {
                const int page = table[new_page];
                if (page >= 0) {
                    float v[4];
                    const bool is_k = warp == WARPS - 2;
                    const int head = is_k ? nq + kvh : nq + nkv + kvh;
                    project_head(pj, row + (size_t)head * HD + lane * 4, is_k ? 1 : 2, t, lane, share, v);
                    __nv_bfloat16* dst = (is_k ? pj.k_out : pj.v_out) +
                                         (((size_t)page * nkv + kvh) * RB_PAGE + (pos % RB_PAGE)) * HD;
                    *reinterpret_cast<uint2*>(dst + lane * 4) = pack4_bf16(v);
                    __threadfence_block();
                }
            }
            __syncthreads();                                // before the page of the new token is copied
        }
        if (!early0) issue(page_first, 0);
        if (!early1) issue(page_first + 1, 1);              // commits an empty group beyond page_last
        for (int r = warp; r < ROWS; r += WARPS) {          // the query heads of this block
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (r < rows_valid) project_head(pj, row + (size_t)(h0 + r) * HD + lane * 4, 0, t, lane, share, v);
            const int chunk = lane >> 1;                    // 8 values per 16-byte chunk, 4 per lane
            *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(Qs) + r * (HD * 2) + ((chunk ^ (r & 7)) << 4) +
                                      (lane & 1) * 8) = pack4_bf16(v);
        }
    } else {
        load_tile<HD>(Qs, q + (size_t)t * q_stride + (size_t)h0 * HD, HD, ROWS, rows_valid, threadIdx.x, WARPS * 32);
    }
    if (!FQ) {
        cp_async_commit();                                  // a group of its own: the wait below covers committed groups only
        if (!early0) issue(page_first, 0);
        if (!early1) issue(page_first + 1, 1);              // commits an empty group beyond page_last
    }
    cp_async_wait<0>();
    __syncthreads();                                        // the query heads are in place for every warp

    float m_w[2] = {NEG_BIG, NEG_BIG}, l_w[2] = {0.f, 0.f};
    // TR: m_w / l_w belong to this lane's two heads (tq * 2, tq * 2 + 1) and `ot` is O^T (tile i: head size
    // i * 16 + gq and + 8 as rows, the two heads as columns); otherwise they belong to the lane's two head
    // rows (gq, gq + 8) and `o` is O.
    float o[TR ? 1 : HD / 8][4];
    float ot[TR ? HD / 16 : 1][4];
    uint32_t qb[TR ? HD / 16 : 1][2];      // TR: the query heads as the B operand, loaded once
#pragma unroll
    for (int i = 0; i < (TR ? 1 : HD / 8); ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
#pragma unroll
    for (int i = 0; i < (TR ? HD / 16 : 1); ++i) { ot[i][0] = ot[i][1] = ot[i][2] = ot[i][3] = 0.f; }
    const uint32_t qs_base = smem_addr(Qs);
    if (TR) {
#pragma unroll
        for (int ks = 0; ks < HD / 16; ks += 2)
            ldmatrix_x4(tile_addr<HD>(qs_base, lane & 7, ks * 2 + (lane >> 3)), qb[ks][0], qb[ks][1], qb[ks + 1][0], qb[ks + 1][1]);
    }
    const float sl2 = scale * LOG2E;

    auto attend_page = [&](int pg, int buf) {
        const int j0 = pg * CHUNK + warp * WK;
        const int hi = min(pos, (pg + 1) * CHUNK - 1);
        if (!(j0 <= hi && j0 + WK - 1 >= win_lo)) return;
        const uint32_t ks_base = smem_addr(KVw + buf * 2 * WK * HD);
        const uint32_t vs_base = ks_base + WK * HD * 2;
        if constexpr (TR) {
            // S^T for the slice's 16 keys: st[0], st[1] = (key gq; heads tq * 2, + 1), st[2], st[3] = (key gq + 8; ...)
            float st[4] = {0.f, 0.f, 0.f, 0.f}, st2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ks = 0; ks < HD / 16; ks += 2) {          // two chains of MMAs, added at the end
                uint32_t ka[4], kb[4];
                const int row = (lane & 7) + ((lane >> 3) & 1) * 8;
                ldmatrix_x4(tile_addr<HD>(ks_base, row, ks * 2 + (lane >> 4)), ka[0], ka[1], ka[2], ka[3]);
                ldmatrix_x4(tile_addr<HD>(ks_base, row, ks * 2 + 2 + (lane >> 4)), kb[0], kb[1], kb[2], kb[3]);
                mma_bf16(st, ka, qb[ks][0], qb[ks][1]);
                mma_bf16(st2, kb, qb[ks + 1][0], qb[ks + 1][1]);
            }
            const int key0 = j0 + gq, key1 = key0 + 8;
            if (j0 >= win_lo && j0 + WK - 1 <= hi) {
#pragma unroll
                for (int e = 0; e < 4; ++e) st[e] = (st[e] + st2[e]) * sl2;
            } else {
                const bool ok0 = key0 >= win_lo && key0 <= hi, ok1 = key1 >= win_lo && key1 <= hi;
                st[0] = ok0 ? (st[0] + st2[0]) * sl2 : -INFINITY;
                st[1] = ok0 ? (st[1] + st2[1]) * sl2 : -INFINITY;
                st[2] = ok1 ? (st[2] + st2[2]) * sl2 : -INFINITY;
                st[3] = ok1 ? (st[3] + st2[3]) * sl2 : -INFINITY;
            }
            float mx[2] = {fmaxf(st[0], st[2]), fmaxf(st[1], st[3])};
            float alpha[2];
            bool moved = false;
#pragma unroll
            for (int r = 0; r < 2; ++r) {                       // a head's keys lie along the lanes' groups
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 4));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 8));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 16));
                const float m_new = fmaxf(m_w[r], mx[r]);
                moved = moved || m_new != m_w[r];
                alpha[r] = ex2(m_w[r] - m_new);
                m_w[r] = m_new;
                l_w[r] *= alpha[r];
            }
            if (pg > page_first && __any_sync(0xffffffffu, moved)) {
#pragma unroll
                for (int i = 0; i < HD / 16; ++i) {
                    ot[i][0] *= alpha[0]; ot[i][1] *= alpha[1];
                    ot[i][2] *= alpha[0]; ot[i][3] *= alpha[1];
                }
            }
            const float p0 = ex2(st[0] - m_w[0]), p1 = ex2(st[1] - m_w[1]);
            const float p2 = ex2(st[2] - m_w[0]), p3 = ex2(st[3] - m_w[1]);
            l_w[0] += p0 + p2;
            l_w[1] += p1 + p3;
            // P as the B operand of O^T = V^T P: (keys tq * 2, + 1; head gq) and the same for keys + 8
            const uint32_t pb0 = movmatrix_trans(pack_bf16(p0, p1));
            const uint32_t pb1 = movmatrix_trans(pack_bf16(p2, p3));
#pragma unroll
            for (int i = 0; i < HD / 16; ++i) {
                uint32_t va[4];
                ldmatrix_x4_trans(tile_addr<HD>(vs_base, (lane & 7) + (lane >> 4) * 8, i * 2 + ((lane >> 3) & 1)),
                                  va[0], va[1], va[2], va[3]);
                mma_bf16(ot[i], va, pb0, pb1);
            }
        } else {
        float s[WK / 8][4];
#pragma unroll
        for (int j = 0; j < WK / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
        for (int ks = 0; ks < HD / 16; ks += 2) {
            uint32_t qa0[4], qa1[4];
            const int row = (lane & 7) + ((lane >> 3) & 1) * 8;
            ldmatrix_x4(tile_addr<HD>(qs_base, row, ks * 2 + (lane >> 4)), qa0[0], qa0[1], qa0[2], qa0[3]);
            ldmatrix_x4(tile_addr<HD>(qs_base, row, ks * 2 + 2 + (lane >> 4)), qa1[0], qa1[1], qa1[2], qa1[3]);
#pragma unroll
            for (int j = 0; j < WK / 8; ++j) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(tile_addr<HD>(ks_base, j * 8 + (lane & 7), ks * 2 + (lane >> 3)), b0, b1, b2, b3);
                mma_bf16(s[j], qa0, b0, b1);
                mma_bf16(s[j], qa1, b2, b3);
            }
        }
        // The kernel is bound by the instructions a warp issues per page, so what a page rarely needs is
        // skipped with a vote: the mask (only a sequence's last page and a window's first can need one;
        // every row is the same token, so one mask serves all rows) and the rescaling of the output
        // (the running maximum seldom moves after the first pages).
        float mx[2] = {NEG_BIG, NEG_BIG};
        if (j0 >= win_lo && j0 + WK - 1 <= hi) {
#pragma unroll
            for (int j = 0; j < WK / 8; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) s[j][e] *= sl2;
                mx[0] = fmaxf(mx[0], fmaxf(s[j][0], s[j][1]));
                mx[1] = fmaxf(mx[1], fmaxf(s[j][2], s[j][3]));
            }
        } else {
#pragma unroll
            for (int j = 0; j < WK / 8; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = j0 + j * 8 + tq * 2 + (e & 1);
                    const bool ok = key >= win_lo && key <= hi;
                    s[j][e] = ok ? s[j][e] * sl2 : -INFINITY;
                }
                mx[0] = fmaxf(mx[0], fmaxf(s[j][0], s[j][1]));
                mx[1] = fmaxf(mx[1], fmaxf(s[j][2], s[j][3]));
            }
        }
        float alpha[2];
        bool moved = false;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_w[r], mx[r]);
            moved = moved || m_new != m_w[r];
            alpha[r] = ex2(m_w[r] - m_new);
            m_w[r] = m_new;
            l_w[r] *= alpha[r];
        }
        if (pg > page_first && __any_sync(0xffffffffu, moved)) {
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) {
                o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
                o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
            }
        }
        uint32_t pa[WK / 16][4];
#pragma unroll
        for (int j = 0; j < WK / 8; ++j) {
            const float p0 = ex2(s[j][0] - m_w[0]), p1 = ex2(s[j][1] - m_w[0]);
            const float p2 = ex2(s[j][2] - m_w[1]), p3 = ex2(s[j][3] - m_w[1]);
            l_w[0] += p0 + p1;
            l_w[1] += p2 + p3;
            pa[j >> 1][(j & 1) * 2] = pack_bf16(p0, p1);
            pa[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
#pragma unroll
        for (int kk = 0; kk < WK / 16; ++kk) {
#pragma unroll
            for (int i = 0; i < HD / 8; i += 2) {
                uint32_t b0, b1, b2, b3;
                const int row = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                ldmatrix_x4_trans(tile_addr<HD>(vs_base, row, i + (lane >> 4)), b0, b1, b2, b3);
                mma_bf16(o[i], pa[kk], b0, b1);
                mma_bf16(o[i + 1], pa[kk], b2, b3);
            }
        }
        }
    };
    for (int pg = page_first; pg <= page_last; ++pg) {
        const int buf = (pg - page_first) & 1;
        if (pg >= page_first + 2) {
            cp_async_wait<1>();                             // page pg has landed; page pg + 1 may be on its way
            __syncwarp();
        }
        attend_page(pg, buf);
        __syncwarp();                                       // the buffer is free again
        issue(pg + 2, buf);
    }
    cp_async_wait<0>();
#pragma unroll
    for (int r = 0; r < 2; ++r) {                           // this thread's share of the sums -> the row's sum
        if (TR) {
            l_w[r] += __shfl_xor_sync(0xffffffffu, l_w[r], 4);
            l_w[r] += __shfl_xor_sync(0xffffffffu, l_w[r], 8);
            l_w[r] += __shfl_xor_sync(0xffffffffu, l_w[r], 16);
        } else {
            l_w[r] += __shfl_xor_sync(0xffffffffu, l_w[r], 1);
            l_w[r] += __shfl_xor_sync(0xffffffffu, l_w[r], 2);
        }
    }
    __syncthreads();   // every warp is done with its keys and values: the space is reused for the merge
    if (TR) {
        if (gq == 0) {
            s_m[warp][tq * 2] = m_w[0]; s_m[warp][tq * 2 + 1] = m_w[1];
            s_l[warp][tq * 2] = l_w[0]; s_l[warp][tq * 2 + 1] = l_w[1];
        }
        const bool h_lo = tq * 2 < rows_valid, h_hi = tq * 2 + 1 < rows_valid;
#pragma unroll
        for (int i = 0; i < HD / 16; ++i) {
            const int d = i * 16 + gq;
            float* lo = s_o + ((size_t)warp * ROWS + tq * 2) * HD + d;
            if (h_lo) { lo[0] = ot[i][0]; lo[8] = ot[i][2]; }
            if (h_hi) { lo[HD] = ot[i][1]; lo[HD + 8] = ot[i][3]; }
        }
    } else if (tq == 0) {
        s_m[warp][gq] = m_w[0]; s_m[warp][gq + 8] = m_w[1];
        s_l[warp][gq] = l_w[0]; s_l[warp][gq + 8] = l_w[1];
    }
    if (!TR) {   // only the rows that hold a query head are read again (a group of 4 fills 4 of the tile's 16 rows)
        const bool lo_row = gq < rows_valid, hi_row = gq + 8 < rows_valid;
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
            const int d = i * 8 + tq * 2;
            if (lo_row) *reinterpret_cast<float2*>(s_o + ((size_t)warp * ROWS + gq) * HD + d) = make_float2(o[i][0], o[i][1]);
            if (hi_row) *reinterpret_cast<float2*>(s_o + ((size_t)warp * ROWS + gq + 8) * HD + d) = make_float2(o[i][2], o[i][3]);
        }
    }
    __syncthreads();
    const size_t row0 = (size_t)b * nq;                   // the work space is indexed by sequence, whatever cu_q says
    for (int idx = threadIdx.x; idx < rows_valid * HD; idx += WARPS * 32) {
        const int r = idx / HD, d = idx % HD;
        float M = NEG_BIG;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) M = fmaxf(M, s_m[w][r]);
        float L = 0.f, A = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float wt = exp2f(s_m[w][r] - M);          // a warp that saw no key has l = 0 and o = 0
            L = fmaf(wt, s_l[w][r], L);
            A = fmaf(wt, s_o[((size_t)w * ROWS + r) * HD + d], A);
        }
        const int head = h0 + r;
        if (CL) {
            s_part[r * HD + d] = A;
            if (d == 0) { s_pm_own[r] = M; s_pl_own[r] = L; }
        } else if (PROP ? parts_hi > 0 : n_chunks > 1) {
            const size_t pidx = (row0 + head) * n_chunks + c;
            part_acc[pidx * HD + d] = A;
            if (d == 0) { part_ml[pidx * 2] = M; part_ml[pidx * 2 + 1] = L; }
        } else {
            out[(size_t)t * o_stride + (size_t)head * HD + d] = __float2bfloat16_rn(L > 0.f ? A / L : 0.f);
        }
    }
    if (CL) {
        // The blocks of this (sequence, head group) are one cluster: each keeps its partial result in
        // its own shared memory, and after a cluster barrier each block merges one slice of the head
        // size, reading every block's part (in ascending order) through distributed shared memory.
        // Nothing goes through global memory, no counter is needed.
        cluster_sync_all();
        const int n = (int)gridDim.x;                        // = the cluster's size, at most MAX_CLUSTER
        const int d_lo = c * HD / n, d_hi = (c + 1) * HD / n;
        const int width = d_hi - d_lo;
        for (int idx = threadIdx.x; idx < rows_valid * width; idx += WARPS * 32) {
            const int r = idx / width, d = d_lo + idx % width;
            // every block's maximum, sum and value for this (row, dimension): all remote reads go out
            // together, one round trip
            float pm[MAX_CLUSTER], pl[MAX_CLUSTER], pa[MAX_CLUSTER];
#pragma unroll
            for (int i = 0; i < MAX_CLUSTER; ++i) {
                if (i < n) {
                    pm[i] = ld_cluster(&s_pm_own[r], (unsigned)i);
                    pl[i] = ld_cluster(&s_pl_own[r], (unsigned)i);
                    pa[i] = ld_cluster(&s_part[r * HD + d], (unsigned)i);
                }
            }
            float MM = NEG_BIG;
#pragma unroll
            for (int i = 0; i < MAX_CLUSTER; ++i)
                if (i < n && pl[i] > 0.f) MM = fmaxf(MM, pm[i]);
            float L = 0.f, A = 0.f;
#pragma unroll
            for (int i = 0; i < MAX_CLUSTER; ++i) {          // in ascending order of the keys
                if (i < n) {
                    const float wt = pl[i] > 0.f ? exp2f(pm[i] - MM) : 0.f;
                    L = fmaf(wt, pl[i], L);
                    A = fmaf(wt, pa[i], A);
                }
            }
            out[(size_t)t * o_stride + (size_t)(h0 + r) * HD + d] = __float2bfloat16_rn(L > 0.f ? A / L : 0.f);
        }
        cluster_sync_all();                                  // nobody leaves while its part may still be read
        return;
    }
    if (PROP ? parts_hi == 0 : n_chunks <= 1) goto round_done;

    // the block that arrives last merges the chunks of this (sequence, head group)
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int active = PROP ? parts_hi + 1 : pos / (CHUNK * ppb) + 1;
        int* ctr = counters + (size_t)b * gridDim.y + blockIdx.y;
        const int old = atomicAdd(ctr, 1);
        s_last = old == active - 1;
        if (s_last) *ctr = 0;              // ready for the next launch
    }
    __syncthreads();
    if (!s_last) goto round_done;
    __threadfence();
    // First every chunk's (maximum, sum) of every row goes to shared memory in one parallel sweep;
    // then each thread owns one (row, dimension) and adds the chunks in ascending order.  Loads of
    // different chunks do not depend on one another, so they overlap.
    const int c_hi = parts_hi, c_lo = parts_lo;
    const int n_act = c_hi - c_lo + 1;
    float* s_pm = reinterpret_cast<float*>(KVs);            // [rows][n_act]
    float* s_pl = s_pm + rows_valid * n_act;            // the host checked that both fit
    for (int idx = threadIdx.x; idx < rows_valid * n_act; idx += WARPS * 32) {
        const int r = idx / n_act, cc = c_lo + idx % n_act;
        const size_t base = (row0 + h0 + r) * n_chunks + cc;
        s_pm[r * n_act + idx % n_act] = __ldcg(part_ml + base * 2);
        s_pl[r * n_act + idx % n_act] = __ldcg(part_ml + base * 2 + 1);
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < rows_valid * HD; idx += WARPS * 32) {
        const int r = idx / HD, d = idx % HD;
        const float* pm = s_pm + r * n_act;
        const float* pl = s_pl + r * n_act;
        float MM = NEG_BIG;
        for (int i = 0; i < n_act; ++i)
            if (pl[i] > 0.f) MM = fmaxf(MM, pm[i]);
        const float* pa = part_acc + ((row0 + h0 + r) * n_chunks + c_lo) * HD + d;
        float L = 0.f, A = 0.f;
#pragma unroll 8
        for (int i = 0; i < n_act; ++i) {
            const float wt = pl[i] > 0.f ? exp2f(pm[i] - MM) : 0.f;
            L = fmaf(wt, pl[i], L);
            A = fmaf(wt, __ldcg(pa + (size_t)i * HD), A);
        }
        out[(size_t)t * o_stride + (size_t)(h0 + r) * HD + d] = __float2bfloat16_rn(L > 0.f ? A / L : 0.f);
    }
   }
round_done:
    if (!PROP) return;
    __syncthreads();                                        // the shared memory is free for the next round
  }
}

bool cluster_enabled() {
    static const bool on = [] {
        const char* v = std::getenv("RB_DECODE_CLUSTER");
        return !(v && v[0] == '0');
    }();
    return on;
}

template <int HD, bool CL, bool FQ, bool PROP, bool TR>
int launch_variant(dim3 grid, size_t smem, cudaStream_t s, const void* q, int q_stride, const void* k_cache,
                   const void* v_cache, const int* block_table, int max_pages, const int* seq_slot, const int* cu_q,
                   const int* kv_len, int nq, int nkv, float scale, int window, int n_chunks, int ppb, float* part_acc,
                   float* part_ml, int* counters, void* out, int o_stride, const Projections& pj, int n_seqs) {
    auto k = attention_decode_kernel<HD, CL, FQ, PROP, TR>;
    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        if (CL) {   // clusters of more than 8 blocks are not portable
            e = cudaFuncSetAttribute(k, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
            if (e != cudaSuccess) return (int)e;
        }
        attr_done = true;
    }
    if (CL) {
        cudaError_t e = launch_clustered(k, grid, dim3(WARPS * 32), dim3(grid.x, 1, 1), smem, s, (const __nv_bfloat16*)q,
                                         q_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
                                         block_table, max_pages, seq_slot, cu_q, kv_len, nq, nkv, scale, window,
                                         n_chunks, ppb, part_acc, part_ml, counters, (__nv_bfloat16*)out, o_stride, pj, n_seqs);
        return e == cudaSuccess ? RB_OK : (int)e;
    } else {
        RB_LAUNCH((k), grid, dim3(WARPS * 32), smem, s, (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache,
                  (const __nv_bfloat16*)v_cache, block_table, max_pages, seq_slot, cu_q, kv_len, nq, nkv, scale, window,
                  n_chunks, ppb, part_acc, part_ml, counters, (__nv_bfloat16*)out, o_stride, pj, n_seqs);
        return RB_OK;
    }
}

template <int HD>
int launch(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int* block_table,
           int max_pages, const int* seq_slot, const int* cu_q, const int* kv_len, int B, int nq, int nkv,
           float scale, int window, int n_chunks, int ppb, float* part_acc, float* part_ml, int* counters,
           void* out, int o_stride, const Projections& pj, cudaStream_t s) {
    const int g = nq / nkv;
    const bool proportional = ppb == 0;     // n_chunks blocks a head group share the pages of all sequences equally
    if (proportional && B > PROP_MAX_SEQS) return RB_ERR_BAD_SIZE;
    dim3 grid(n_chunks, nkv * ((g + ROWS - 1) / ROWS), proportional ? 1 : B);
    if (grid.y > 65535 || grid.z > 65535) return RB_ERR_BAD_SIZE;
    const size_t kv_bytes = (size_t)WARPS * 4 * WK * HD * sizeof(__nv_bfloat16);   // two buffers per warp
    const size_t merge_bytes = (size_t)WARPS * ROWS * HD * sizeof(float);
    const size_t smem = (size_t)ROWS * HD * sizeof(__nv_bfloat16) + (kv_bytes > merge_bytes ? kv_bytes : merge_bytes);
    const size_t region = kv_bytes > merge_bytes ? kv_bytes : merge_bytes;
    const int rows_max = g < ROWS ? g : ROWS;
    if ((size_t)n_chunks * rows_max * 2 * sizeof(float) > region) return RB_ERR_BAD_SIZE;  // the merge's work space
    // up to 16 blocks per (sequence, head group): one cluster, merged through shared memory
    const bool clustered = !proportional && n_chunks > 1 && n_chunks <= MAX_CLUSTER && cluster_enabled();
    const bool fused = pj.proj != nullptr;
    if (fused && HD != 128) return RB_ERR_BAD_SIZE;
    // More than 16 query heads a key/value head: several blocks read the page of the new token, and only
    // one of them writes the token's key and value into it, with nothing that orders the others' reads
    // after that write.  The caller writes the cache with the kernel of its own and calls again.
    if (fused && pj.write_kv && g > ROWS) return RB_ERR_BAD_SIZE;
    // groups of up to 8 heads (every size of the architecture): the transposed products (see the kernel)
#define RB_ADV(CL, FQ, PROP) (g <= 8 ? launch_variant<HD, CL, FQ, PROP, true>(grid, smem, s, q, q_stride, k_cache, v_cache, block_table, \
                                                         max_pages, seq_slot, cu_q, kv_len, nq, nkv, scale, window,         \
                                                         n_chunks, ppb, part_acc, part_ml, counters, out, o_stride, pj, B)  \
                                     : launch_variant<HD, CL, FQ, PROP, false>(grid, smem, s, q, q_stride, k_cache, v_cache, block_table, \
                                                         max_pages, seq_slot, cu_q, kv_len, nq, nkv, scale, window,         \
                                                         n_chunks, ppb, part_acc, part_ml, counters, out, o_stride, pj, B))
    if (proportional) return (HD == 128 && fused) ? RB_ADV(false, (HD == 128), true) : RB_ADV(false, false, true);
    if (HD == 128 && fused) return clustered ? RB_ADV(true, (HD == 128), false) : RB_ADV(false, (HD == 128), false);
    return clustered ? RB_ADV(true, false, false) : RB_ADV(false, false, false);
#undef RB_ADV
}
}  // namespace

// One query token per sequence (token index cu_q[b]).  A block takes `pages_per_block` pages of 64
// keys; n_chunks = ceil(pages of the longest sequence / pages_per_block) blocks cover a sequence;
// with n_chunks == 1 the result is written to `out` directly.  pages_per_block == 0: n_chunks blocks
// per key/value head group share the pages of all B sequences (B <= 256) equally, a block working on
// the end of one sequence and the beginning of the next where its share says so.
// Work space: part_acc [B, nq, n_chunks, hd], part_ml [B, nq, n_chunks, 2] (indexed by the sequence's
// place in the batch, not by its token index) and `counters`, at least
// B * nkv * ceil(group / 16) ints that are ZERO on entry and are left zero on exit.
// Returns RB_ERR_BAD_SIZE for head sizes other than 64, 128, 256 and for contexts whose chunk list does
// not fit the merge's shared memory (65536 tokens at a group of 4 and head size 128); the caller then
// uses the plain kernel.
static int decode_entry(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                        const int* block_table, int max_pages, const int* seq_slot, const int* cu_q,
                        const int* kv_len, int B, int nq, int nkv, int hd, float scale, int window,
                        int n_chunks, int pages_per_block, float* part_acc, float* part_ml,
                        int* counters, void* out, int o_stride, const Projections& pj, void* stream) {
    if (B <= 0) return RB_OK;
    if (nkv <= 0 || nq % nkv || n_chunks < 1 || n_chunks > 1024 || pages_per_block < 0) return RB_ERR_BAD_SIZE;
    if (n_chunks > 1 && (!part_acc || !part_ml || !counters)) return RB_ERR_BAD_SIZE;
    if (((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15)) return RB_ERR_BAD_ALIGN;
    if (pj.proj == nullptr && (((uintptr_t)q & 15) || (q_stride % 8))) return RB_ERR_BAD_ALIGN;
    cudaStream_t s = (cudaStream_t)stream;
#define RB_AD(HD) return launch<HD>(q, q_stride, k_cache, v_cache, block_table, max_pages, seq_slot, cu_q, kv_len, B, nq, \
                                    nkv, scale, window, n_chunks, pages_per_block, part_acc, part_ml, counters, out, o_stride, pj, s)
    if (hd == 128) RB_AD(128);
    if (hd == 64) RB_AD(64);
    if (hd == 256) RB_AD(256);
#undef RB_AD
    return RB_ERR_BAD_SIZE;
}

extern "C" int rb_attention_decode(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                   const int* block_table, int max_pages, const int* seq_slot, const int* cu_q,
                                   const int* kv_len, int B, int nq, int nkv, int hd, float scale, int window,
                                   int n_chunks, int pages_per_block, float* part_acc, float* part_ml,
                                   int* counters, void* out, int o_stride, void* stream) {
    Projections none = {};
    return decode_entry(q, q_stride, k_cache, v_cache, block_table, max_pages, seq_slot, cu_q, kv_len, B, nq, nkv, hd,
                        scale, window, n_chunks, pages_per_block, part_acc, part_ml, counters, out, o_stride, none, stream);
}

// The same for head size 128 with the step's projections as the matrix product left them:
// proj [n_in][T][(nq + 2 * nkv) * 128] float32 partial sums (queries, keys, values side by side;
// in_stride elements between partial sums, row_stride between tokens; with write_kv == 0 only the
// nq query heads are there).  The kernel adds them, normalises (norm weights [128], float32 if
// w_f32 else bfloat16, or null) and rotates (cos_sin [T][64] pairs, or null) the query heads itself,
// and writes the new token's key and value into the cache (write_kv != 0) before reading it.
// With row_sumsq (shares [row_groups][>= T] of the sums of squares of the rows the projection was made
// from, over row_width values each) the sums are first scaled by rsqrt(sum / row_width + row_eps).
// Returns RB_ERR_BAD_SIZE for other head sizes, RB_ERR_BAD_ALIGN for partial sums off 16 bytes.
extern "C" int rb_attention_decode_fused(const float* proj, int n_in, long long in_stride, int row_stride,
                                         const void* q_norm_w, const void* k_norm_w, int w_f32, float eps,
                                         const float* cos_sin, int write_kv, const float* row_sumsq, int row_groups,
                                         long long row_sumsq_ld, float row_eps, int row_width,
                                         void* k_cache, void* v_cache,
                                         const int* block_table, int max_pages, const int* seq_slot, const int* cu_q,
                                         const int* kv_len, int B, int nq, int nkv, int hd, float scale, int window,
                                         int n_chunks, int pages_per_block, float* part_acc, float* part_ml,
                                         int* counters, void* out, int o_stride, void* stream) {
    if (hd != 128 || proj == nullptr || n_in < 1) return RB_ERR_BAD_SIZE;
    if (((uintptr_t)proj & 15) || (in_stride % 4) || (row_stride % 4) || ((uintptr_t)cos_sin & 7)) return RB_ERR_BAD_ALIGN;
    if ((q_norm_w == nullptr) != (k_norm_w == nullptr)) return RB_ERR_BAD_SIZE;
    Projections pj;
    pj.proj = proj; pj.n_in = n_in; pj.in_stride = in_stride; pj.row_stride = row_stride;
    pj.q_norm_w = q_norm_w; pj.k_norm_w = k_norm_w; pj.w_f32 = w_f32; pj.eps = eps;
    pj.cos_sin = reinterpret_cast<const float2*>(cos_sin);
    pj.write_kv = write_kv;
    pj.k_out = static_cast<__nv_bfloat16*>(k_cache);
    pj.v_out = static_cast<__nv_bfloat16*>(v_cache);
    pj.row_sumsq = row_sumsq; pj.row_groups = row_groups; pj.row_sumsq_ld = row_sumsq_ld;
    pj.row_eps = row_eps; pj.row_inv_width = row_width > 0 ? 1.f / (float)row_width : 0.f;
    if (row_sumsq != nullptr && (row_groups < 1 || row_width < 1)) return RB_ERR_BAD_SIZE;
    return decode_entry(nullptr, 0, k_cache, v_cache, block_table, max_pages, seq_slot, cu_q, kv_len, B, nq, nkv, hd,
                        scale, window, n_chunks, pages_per_block, part_acc, part_ml, counters, out, o_stride, pj, stream);
}

// ---- the same kernel for callers that cannot allocate (see no_alloc.h) -----------------------------
#include "no_alloc.h"
#include <cstdio>
#include <mutex>

namespace {
constexpr size_t STATIC_ACC_FLOATS = 4u << 20;     // 16 MiB
constexpr size_t STATIC_ML_FLOATS = 256u << 10;    // 1 MiB
constexpr size_t STATIC_COUNTERS = 16u << 10;      // 64 KiB
struct StaticScratch {
    float acc[STATIC_ACC_FLOATS];
    float ml[STATIC_ML_FLOATS];
    int counters[STATIC_COUNTERS];
};
// Part of the device image: every GPU that loads the library holds it until the process exits.
// In host code this name is only a handle for cudaGetSymbolAddress, never an address to pass on.
static __device__ __align__(256) StaticScratch g_static_scratch;

constexpr int MAX_DEVICES = 64;
StaticScratch* g_scratch_addr[MAX_DEVICES] = {};
std::mutex g_scratch_mu;

// The array's address on the current device, looked up once per device.
int static_scratch(StaticScratch** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= MAX_DEVICES) return RB_ERR_BAD_SIZE;
    std::lock_guard<std::mutex> g(g_scratch_mu);
    if (!g_scratch_addr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return (int)e;
        g_scratch_addr[dev] = static_cast<StaticScratch*>(p);
    }
    *out = g_scratch_addr[dev];
    return RB_OK;
}
}  // namespace

extern "C" int rb_attention_decode_static(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                          const int* block_table, int max_pages, const int* seq_slot,
                                          const int* cu_q, const int* kv_len, int n_seqs, int nq, int nkv, int hd,
                                          float scale, int window, int n_chunks, void* out, int o_stride,
                                          void* stream) {
    if (n_seqs <= 0) return RB_OK;
    if (nkv <= 0 || nq <= 0 || nq % nkv || hd <= 0 || n_chunks < 1) return RB_ERR_BAD_SIZE;
    const size_t rows = (size_t)n_seqs * nq * n_chunks;
    const size_t n_counters = (size_t)n_seqs * nkv * ((nq / nkv + ROWS - 1) / ROWS);
    if (rows * hd > STATIC_ACC_FLOATS || rows * 2 > STATIC_ML_FLOATS || n_counters > STATIC_COUNTERS) {
        std::fprintf(stderr,
                     "rb_attention_decode_static: %d sequences x %d heads x %d chunks x head size %d needs %zu partial "
                     "floats (limit %zu), %zu max/sum floats (limit %zu), %zu counters (limit %zu)\n",
                     n_seqs, nq, n_chunks, hd, rows * hd, STATIC_ACC_FLOATS, rows * 2, STATIC_ML_FLOATS, n_counters,
                     STATIC_COUNTERS);
        return RB_ERR_SCRATCH_LIMIT;
    }
    StaticScratch* sc = nullptr;
    int rc = static_scratch(&sc);
    if (rc != RB_OK) return rc;
    // the counters must start at zero whatever an earlier call left behind
    cudaError_t e = cudaMemsetAsync(sc->counters, 0, n_counters * sizeof(int), (cudaStream_t)stream);
    if (e != cudaSuccess) return (int)e;
    return rb_attention_decode(q, q_stride, k_cache, v_cache, block_table, max_pages, seq_slot, cu_q, kv_len, n_seqs,
                               nq, nkv, hd, scale, window, n_chunks, 1, sc->acc, sc->ml, sc->counters, out, o_stride,
                               stream);
}
