// Flash attention for bfloat16 prompts over the paged cache on the 5th-generation tensor cores:
// S = Q K^T and O += P V are tcgen05.mma with the accumulators in tensor memory; Q, K and V tiles
// arrive by TMA; the softmax runs in registers, one thread per query row (a TMEM lane is a row, so no
// shuffles are needed for row maxima and sums).  Head sizes 64, 128 and 256 (a template argument).
//
// A block takes 128 query tokens of one sequence and one query head and walks the keys page by page
// (a page of the cache is one 64-key tile).  Roles: warp 0 issues TMA loads (Q once, K and V in rings
// of two, so that a tile's copies never wait for the products of the tile before), warp 1 issues
// the MMAs, warps 2-5 are the 128 softmax threads.
// Per tile: S_j = Q K_j^T into one of two TMEM buffers (so the tensor core can already form S_{j+1}
// while the softmax works on S_j); the softmax threads read their row, mask (causal, inclusive;
// window), update the running maximum and sum in float32 (base 2, the scale folded into the
// exponent's multiply-add, two scores an instruction), and write P as pairs of bfloat16 back into
// the first 32 columns of the buffer S_j came from: the tensor core reads its A operand from there
// (no shared-memory round trip, no proxy fence; S_{j+2} is issued into that buffer after the product
// that reads P_j from it, see `strict_order` in the MMA thread).  Only when some row's maximum has grown by
// more than 2^8 does a warp wait for the last product and rescale the O accumulator in tensor memory
// (otherwise the stale maximum stays in use, which is exact: numerator and denominator carry the
// same factor); O += P V_j with V read in its natural [key][dimension] order (MN-major operand).
// Up to head size 128 two blocks share a multiprocessor (112 KB of shared memory and 256 TMEM columns
// each), so one block's softmax overlaps the other's MMAs; at head size 256 a block's tiles take 192 KB
// and its accumulators 384 columns, so it is alone.
//
// Same mathematics as the reference's attn_prefill_flash_* (rocml-kernels/kernels/
// attn_prefill_flash_impl.h:46-159): head h reads key/value head h / g, score = (q.k) * scale, query
// at position p sees keys 0..p, online softmax, o = sum p v / l.  Every wait is bounded.
#include "common.cuh"
#include "sm100.cuh"
#include "api.h"
#include <stdlib.h>
#include <mutex>
#include <unordered_map>

using namespace sm100;

namespace {
constexpr int BMQ = 128;      // query rows per block
constexpr int BNK = 64;       // keys per tile = one page
constexpr float LOG2E = 1.4426950408889634f;
constexpr float NEG_BIG = -1e30f;
constexpr float RESCALE_AT = 8.0f;   // rescale O when a row maximum grew by more than 2^8

// What depends on the head size (64, 128 or 256): every tile is HD / 64 blocks of 64 dimensions (128 bytes a row,
// 128-byte swizzle), one TMA box each.
template <int HD>
struct Sizes {
    static constexpr int HALVES = HD / 64;                 // 64-dimension blocks a row
    static constexpr int Q_BYTES = BMQ * HD * 2;           // Q: HALVES x [128 rows][64]; 32 KB at head size 128
    static constexpr int KV_TILE = BNK * HD * 2;           // K or V: HALVES x [64 keys][64]; 16 KB at head size 128
    static constexpr int Q_HALF = Q_BYTES / HALVES, KV_HALF = KV_TILE / HALVES;
    static constexpr int TILE_BYTES = Q_BYTES + 2 * KV_TILE + 2 * KV_TILE;     // K and V in rings of two
    // Up to head size 128 two blocks share a multiprocessor's 228 KB (each block is charged 1 KB on top of what
    // it asks for) and its 512 tensor-memory columns; what is left of the allowance is slack for aligning
    // the tiles to 1 KB (the launch's shared memory normally starts on such a boundary; the kernel checks).
    static constexpr int BLOCKS_PER_SM = HD <= 128 ? 2 : 1;
    static constexpr int SMEM_BYTES = BLOCKS_PER_SM == 2 ? (228 * 1024) / 2 - 1024 : TILE_BYTES + 2048;
    static_assert(SMEM_BYTES >= TILE_BYTES + 1024 + 128, "the tiles, their alignment and the barriers must fit");
    // tensor memory columns: S0 [0, 64), S1 [64, 128), O [128, 128 + HD)
    static constexpr int TMEM_COLS = HD <= 128 ? 256 : 512;
};

// 2^x on the special-function unit, one instruction (x <= 0 here, -inf gives 0); the library's exp2f
// adds range handling that the softmax does not need.
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Two float32 operations in one instruction (sm_100): the softmax threads are bound by the instructions
// they issue, and a pair of neighbouring scores sits in a pair of neighbouring registers anyway.
__device__ __forceinline__ uint64_t pack2(float a, float b) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& a, float& b) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// A softmax thread's wait: the flag that another role raises when its own wait ran out is only looked at
// while the barrier is not yet complete (the usual case finds it complete and pays for nothing else).
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, const uint32_t* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (*(volatile const uint32_t*)abort_flag != 0 || clock64() - t0 > RB_WAIT_CYCLES) return false;
    }
    return true;
}

struct Barriers {
    uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full[2], o_done, o_final;
    uint32_t tmem_slot, abort_flag;
};

template <int HD>
__global__ void __launch_bounds__(192, Sizes<HD>::BLOCKS_PER_SM)
attention_prefill_tc5_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                             const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out, int o_stride,
                             const int* __restrict__ block_table, int max_pages, const int* __restrict__ seq_slot,
                             const int* __restrict__ cu_q, const int* __restrict__ kv_len, int nq, int nkv,
                             float scale, int window, int heads_first, int strict_order, int* __restrict__ status) {
    using Z = Sizes<HD>;
    constexpr int HALVES = Z::HALVES, Q_BYTES = Z::Q_BYTES, KV_TILE = Z::KV_TILE, Q_HALF = Z::Q_HALF, KV_HALF = Z::KV_HALF;
    constexpr int TILE_BYTES = Z::TILE_BYTES, SMEM_BYTES = Z::SMEM_BYTES, TMEM_COLS = Z::TMEM_COLS;
    rb::pdl_trigger();
    rb::pdl_wait();
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    if (smem + TILE_BYTES + sizeof(Barriers) > smem_raw + SMEM_BYTES) {   // never seen: the window starts on 1 KB
        if (threadIdx.x == 0) atomicExch(status, RB_ERR_BAD_ALIGN);
        return;
    }
    uint8_t* Qs = smem;
    uint8_t* Ks = Qs + Q_BYTES;               // [2 stages][16 KB]
    uint8_t* Vs = Ks + 2 * KV_TILE;
    Barriers* bar = (Barriers*)(Vs + 2 * KV_TILE);   // V: [2 stages][16 KB]

    // Blocks are handed out with x running fastest.  The last query tiles see the most keys and start
    // first.  heads_first, grid = (heads, sequences, query tiles): the long blocks of ALL heads and
    // sequences start first and the short ones fill the grid's tail (one head's tiles after another's
    // leave a long block of the last head to the end).  Otherwise grid = (query tiles, heads, sequences):
    // the blocks that run together read the keys and values of one or two heads, which matters once
    // all heads' keys and values together no longer fit the L2 cache.
    const int b = heads_first ? blockIdx.y : blockIdx.z, head = heads_first ? blockIdx.x : blockIdx.y;
    const int slot = seq_slot[b];
    const int q0 = cu_q[b], q_len = cu_q[b + 1] - q0;
    const int m0 = heads_first ? (int)(gridDim.z - 1 - blockIdx.z) * BMQ : (int)(gridDim.x - 1 - blockIdx.x) * BMQ;
    if (slot < 0 || m0 >= q_len) return;
    const int len = kv_len[b];
    const int pos0 = len - q_len;
    const int kvh = head / (nq / nkv);
    const int rows_here = min(BMQ, q_len - m0);
    const int hi = pos0 + m0 + rows_here - 1;
    const int lo = window > 0 ? max(0, pos0 + m0 - window + 1) : 0;
    const int kt_first = lo / BNK, kt_last = hi / BNK;
    const int n_tiles = kt_last - kt_first + 1;
    const int* table = block_table + (size_t)slot * max_pages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(&bar->q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bar->k_full[i], 1); mbar_init(&bar->k_empty[i], 1); mbar_init(&bar->s_full[i], 1);
            mbar_init(&bar->v_full[i], 1); mbar_init(&bar->v_empty[i], 1);
        }
        mbar_init(&bar->p_full[0], 128);
        mbar_init(&bar->p_full[1], 128);
        mbar_init(&bar->o_done, 1);
        mbar_init(&bar->o_final, 1);
        bar->abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(&bar->tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = bar->tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            tma_prefetch_desc(&map_q);
            tma_prefetch_desc(&map_k);
            tma_prefetch_desc(&map_v);
            mbar_arrive_expect_tx(&bar->q_full, Q_BYTES);
#pragma unroll
            for (int h = 0; h < HALVES; ++h) tma_load_2d(Qs + h * Q_HALF, &map_q, head * HD + h * 64, q0 + m0, &bar->q_full);
            bool ok = true;
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int page = table[kt_first + j];
                const int row = ((page < 0 ? 0 : page) * nkv + kvh) * RB_PAGE;
                const int s = j & 1;
                ok = mbar_wait(&bar->k_empty[s], ((j >> 1) & 1) ^ 1);
                if (!ok) break;
                mbar_arrive_expect_tx(&bar->k_full[s], KV_TILE);
#pragma unroll
                for (int h = 0; h < HALVES; ++h) tma_load_2d(Ks + s * KV_TILE + h * KV_HALF, &map_k, h * 64, row, &bar->k_full[s]);
                ok = mbar_wait(&bar->v_empty[s], ((j >> 1) & 1) ^ 1);
                if (!ok) break;
                mbar_arrive_expect_tx(&bar->v_full[s], KV_TILE);
#pragma unroll
                for (int h = 0; h < HALVES; ++h) tma_load_2d(Vs + s * KV_TILE + h * KV_HALF, &map_v, h * 64, row, &bar->v_full[s]);
            }
            if (!ok) { atomicExch(status, RB_ERR_TIMEOUT); atomicExch(&bar->abort_flag, 1u); }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_s = idesc_bf16_f32(BMQ, BNK);          // S = Q K^T: both K-major
            constexpr uint32_t idesc_o = idesc_bf16_f32_b_mn(BMQ, HD);      // O += P V: V is MN-major
            // This lone thread executes a dependent instruction every few cycles at best, and a tile's twelve
            // MMAs take the tensor core only 640 cycles: the descriptors are kept as low words that differ
            // from MMA to MMA by constants (sm100.cuh: mma_bf16_lo), not built anew each time.
            const uint32_t q_lo = smem_desc_sw128_lo(smem_u32(Qs)), k_lo0 = smem_desc_sw128_lo(smem_u32(Ks));
            // V is MN-major: leading byte offset = the distance between its two 64-dimension blocks
            const uint32_t v_lo0 = ((smem_u32(Vs) >> 4) & 0x3FFFu) | ((uint32_t)(KV_HALF >> 4) << 16);
            auto issue_s = [&](int j) -> bool {
                const int s = j & 1;
                // S_j goes into the buffer that still holds P_{j-2}, which the product O += P_{j-2} V reads: that
                // product must be DONE, not just issued.  MMAs of one thread are only sure to run in issue order
                // when they write the same accumulator with the same shape, and this one writes S while that one
                // wrote O.  (Without the wait, 280 launches over seven shapes gave the same bits every time and
                // the kernel was 1 to 2 % quicker: the tensor core does take them in order today.
                // RB_PREFILL_STRICT_ORDER=0 leaves the wait out.)
                if (strict_order && j >= 2 && !mbar_wait(&bar->o_done, (j - 2) & 1)) return false;
                if (!mbar_wait(&bar->k_full[s], (j >> 1) & 1)) return false;
                tc_fence_after();
                const uint32_t k_lo = k_lo0 + s * (KV_TILE >> 4);
                const uint32_t d = tmem_base + s * BNK;
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    // dimension block k / 4 (64 dimensions each), 32 bytes (2 units of 16) per step inside it
                    const uint32_t qo = (k >> 2) * (Q_HALF >> 4) + (k & 3) * 2;
                    const uint32_t ko = (k >> 2) * (KV_HALF >> 4) + (k & 3) * 2;
                    mma_bf16_lo(d, q_lo + qo, k_lo + ko, idesc_s, k > 0 ? 1u : 0u);
                }
                mma_commit(&bar->k_empty[s]);
                mma_commit(&bar->s_full[s]);
                return true;
            };
            bool ok = mbar_wait(&bar->q_full, 0);
            if (ok) { tc_fence_after(); ok = issue_s(0); }
            for (int j = 0; j < n_tiles && ok; ++j) {
                if (j + 1 < n_tiles) { ok = issue_s(j + 1); if (!ok) break; }
                ok = mbar_wait(&bar->p_full[j & 1], (j >> 1) & 1) && mbar_wait(&bar->v_full[j & 1], (j >> 1) & 1);
                if (!ok) break;
                tc_fence_after();
                const uint32_t v_lo = v_lo0 + (j & 1) * (KV_TILE >> 4);
#pragma unroll
                for (int k = 0; k < BNK / 16; ++k) {
                    // A = P [128 rows][64 keys] in tensor memory, where S_j was: 16 keys = 8 columns.  B = V [64 keys]
                    // [128 dims], MN-major: 64-dimension blocks 8 KB apart, groups of 8 keys 1 KB apart, 16 keys = 2 KB.
                    mma_bf16_ts_lo(tmem_base + 2 * BNK, tmem_base + (j & 1) * BNK + k * 8, v_lo + k * (2048 >> 4), idesc_o,
                                   (j > 0 || k > 0) ? 1u : 0u);
                }
                mma_commit(&bar->v_empty[j & 1]);
                mma_commit(&bar->o_done);
                // The softmax threads wait for O only when they rescale it, so at the end they may be two
                // phases behind o_done, which a parity cannot tell apart: the last product has a barrier of its own.
                if (j == n_tiles - 1) mma_commit(&bar->o_final);
            }
            if (!ok) {
                atomicExch(status, RB_ERR_TIMEOUT);
                atomicExch(&bar->abort_flag, 1u);      // the softmax threads' waits see it and give up
            }
        }
    } else {
        // softmax: thread r owns query row r (TMEM lane r)
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const int row_pos = pos0 + m0 + r;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const float sl2 = scale * LOG2E;
        float m_used = NEG_BIG, l_sum = 0.f;
        bool alive = true;
        for (int j = 0; j < n_tiles; ++j) {
            const int s = j & 1;
            alive = __all_sync(0xffffffffu, wait_or_abort(&bar->s_full[s], (j >> 1) & 1, &bar->abort_flag));
            if (!alive) break;
            tc_fence_after();
            const int key0 = (kt_first + j) * BNK;
            float sv[BNK];
            static_assert(BNK == 64, "one load of 64 columns");
            tmem_ld64(lane_base + s * BNK, sv);
            // The softmax threads are bound by the instructions they issue.  Scores stay raw: the scale is
            // positive, so the maximum is taken first (three inputs an instruction) and the scale is
            // folded into the exponent's multiply-add, p = 2^(s * scale * log2 e - m), with the bare
            // special-function instruction for 2^x.
            // a tile that every row of this warp sees whole needs no mask
            const int warp_first_pos = pos0 + m0 + quarter * 32;
            if (!(key0 + BNK - 1 <= warp_first_pos && (window <= 0 || key0 > warp_first_pos + 31 - window))) {
#pragma unroll
                for (int i = 0; i < BNK; ++i) {
                    const int key = key0 + i;
                    const bool ok = key <= row_pos && (window <= 0 || key > row_pos - window);
                    sv[i] = ok ? sv[i] : -INFINITY;
                }
            }
            // four chains of maxima side by side (three inputs an instruction)
            float mxa[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) mxa[q] = fmaxf(sv[2 * q], sv[2 * q + 1]);
#pragma unroll
            for (int i = 8; i < BNK; i += 8) {
#pragma unroll
                for (int q = 0; q < 4; ++q) mxa[q] = max3(mxa[q], sv[i + 2 * q], sv[i + 2 * q + 1]);
            }
            const float mx = fmaxf(fmaxf(mxa[0], mxa[1]), fmaxf(mxa[2], mxa[3])) * sl2;
            // the maximum in use only moves when it would otherwise let p exceed 2^8
            const bool grow = mx - m_used > RESCALE_AT;
            const float m_new = grow ? mx : m_used;
            const float alpha = ex2(m_used - m_new);            // 1 when the maximum stays
            m_used = m_new;
            l_sum *= alpha;
            // O is only touched when some row's maximum moved, and only then must the last product be done
            if (j > 0 && __any_sync(0xffffffffu, grow)) {
                alive = __all_sync(0xffffffffu, wait_or_abort(&bar->o_done, (j - 1) & 1, &bar->abort_flag));
                if (!alive) break;
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < HD / 16; ++c) {
                    float ov[16];
                    tmem_ld16(lane_base + 2 * BNK + c * 16, ov);
#pragma unroll
                    for (int i = 0; i < 16; ++i) ov[i] *= alpha;
                    tmem_st16(lane_base + 2 * BNK + c * 16, ov);
                }
            }
            // p = 2^(s * scale * log2 e - m), two at a time; P goes back into the columns S_j came from, as pairs
            // of bfloat16, and the tensor core reads it from there
            const uint64_t sl2_2 = pack2(sl2, sl2), neg_m2 = pack2(-m_used, -m_used);
            uint64_t lacc[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
            for (int c = 0; c < BNK / 32; ++c) {
                uint32_t packed[16];
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    float x0, x1;
                    unpack2(fma2(pack2(sv[c * 32 + e], sv[c * 32 + e + 1]), sl2_2, neg_m2), x0, x1);
                    const float p0 = ex2(x0), p1 = ex2(x1);
                    lacc[(e >> 1) & 3] = add2(lacc[(e >> 1) & 3], pack2(p0, p1));
                    __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                    packed[e / 2] = *reinterpret_cast<uint32_t*>(&h);
                }
                tmem_st16u(lane_base + s * BNK + c * 16, packed);
            }
            float l0, l1;
            unpack2(add2(add2(lacc[0], lacc[1]), add2(lacc[2], lacc[3])), l0, l1);
            l_sum += l0 + l1;
            // the last tile may reach past the sequence's end: what lies there in the page is not ours, and
            // a stale NaN times a zero probability would still poison the sum, so those V rows are zeroed
            // (after the tile has landed, before the product reads it)
            if (j == n_tiles - 1) {
                const int valid = min(BNK, len - key0);
                if (valid < BNK) {
                    alive = __all_sync(0xffffffffu, wait_or_abort(&bar->v_full[j & 1], (j >> 1) & 1, &bar->abort_flag));
                    if (!alive) break;
                    uint8_t* Vt = Vs + (j & 1) * KV_TILE;
                    constexpr int CHUNKS = HD / 8;       // 16-byte chunks of a row of HD bfloat16
                    for (int idx = threadIdx.x - 64; idx < (BNK - valid) * CHUNKS; idx += 128) {
                        const int vr = valid + idx / CHUNKS, ch = idx % CHUNKS;   // row vr, chunk ch of its HD * 2 bytes
                        *reinterpret_cast<uint4*>(Vt + (ch >> 3) * KV_HALF + vr * 128 + (((ch & 7) ^ (vr & 7)) << 4)) =
                            make_uint4(0, 0, 0, 0);
                    }
                    fence_proxy_async();         // shared-memory writes become visible to the tensor core
                }
            }
            tmem_st_wait();
            tc_fence_before();
            // A warp may be a tile ahead of another (S_{j+1} is there before the other has handed P_j over; a warp
            // that needs no mask and no rescaling is quicker), never two (S_{j+2} follows the product of P_j): the
            // arrivals of even and odd tiles are counted apart, or the quick warp's next arrival would complete
            // this tile's count while the slow warp's rows of P are still missing.
            mbar_arrive(&bar->p_full[j & 1]);
        }
        if (alive) alive = __all_sync(0xffffffffu, wait_or_abort(&bar->o_final, 0, &bar->abort_flag));
        if (alive) {
            tc_fence_after();
            const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
            __nv_bfloat16* orow = out + (size_t)(q0 + m0 + r) * o_stride + (size_t)head * HD;
#pragma unroll 1
            for (int c = 0; c < HD / 16; ++c) {
                float ov[16];
                tmem_ld16(lane_base + 2 * BNK + c * 16, ov);
                if (r < rows_here) {
                    uint32_t w[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        __nv_bfloat162 h = __floats2bfloat162_rn(ov[2 * i] * inv, ov[2 * i + 1] * inv);
                        w[i] = *reinterpret_cast<uint32_t*>(&h);
                    }
                    reinterpret_cast<uint4*>(orow + c * 16)[0] = make_uint4(w[0], w[1], w[2], w[3]);
                    reinterpret_cast<uint4*>(orow + c * 16)[1] = make_uint4(w[4], w[5], w[6], w[7]);
                }
            }
        } else if (lane == 0) {
            atomicExch(status, RB_ERR_TIMEOUT);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

// [rows, cols] bf16 with row stride ld (elements), read in boxes of box_rows x 64 columns, 128-byte swizzle.
int make_map(const void* ptr, long long rows, long long cols, long long ld, int box_rows, CUtensorMap* out) {
    struct Key {
        const void* p; long long r, c, l; int b;
        bool operator==(const Key& o) const { return p == o.p && r == o.r && c == o.c && l == o.l && b == o.b; }
    };
    struct Hash {
        size_t operator()(const Key& k) const {
            return ((((size_t)k.p * 1000003u ^ (size_t)k.r) * 1000003u ^ (size_t)k.c) * 1000003u ^ (size_t)k.l) * 31u + k.b;
        }
    };
    static std::mutex mu;
    static std::unordered_map<Key, CUtensorMap, Hash> cache;
    Key key{ptr, rows, cols, ld, box_rows};
    {
        std::lock_guard<std::mutex> g(mu);
        auto it = cache.find(key);
        if (it != cache.end()) { *out = it->second; return RB_OK; }
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return RB_ERR_NO_DRIVER_FN;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    if (fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return RB_ERR_BAD_SIZE;
    std::lock_guard<std::mutex> g(mu);
    if (cache.size() > 65536) cache.clear();
    cache[key] = *out;
    return RB_OK;
}
template <int HD>
int launch_tc5(const void* q, int q_stride, int T, void* out, int o_stride, const void* k_cache, const void* v_cache,
               int n_pages, const int* block_table, int max_pages, const int* seq_slot, const int* cu_q,
               const int* kv_len, int B, int max_q_len, int nq, int nkv, float scale, int window, int heads_first,
               int* status, cudaStream_t stream) {
    // RB_PREFILL_STRICT_ORDER=0: see `strict_order` in the kernel's MMA thread
    static const int strict_order = [] { const char* e = getenv("RB_PREFILL_STRICT_ORDER"); return (e && e[0] == '0') ? 0 : 1; }();
    CUtensorMap mq, mk, mv;
    int rc;
    if ((rc = make_map(q, T, (long long)nq * HD, q_stride, BMQ, &mq)) != RB_OK) return rc;
    const long long cache_rows = (long long)n_pages * nkv * RB_PAGE;
    if ((rc = make_map(k_cache, cache_rows, HD, HD, BNK, &mk)) != RB_OK) return rc;
    if ((rc = make_map(v_cache, cache_rows, HD, HD, BNK, &mv)) != RB_OK) return rc;
    auto k = attention_prefill_tc5_kernel<HD>;
    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, Sizes<HD>::SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        attr_done = true;
    }
    const int q_tiles = (max_q_len + BMQ - 1) / BMQ;
    dim3 grid = heads_first ? dim3(nq, B, q_tiles) : dim3(q_tiles, nq, B);
    if (grid.y > 65535 || grid.z > 65535) return RB_ERR_BAD_SIZE;
    RB_LAUNCH((k), grid, dim3(192), Sizes<HD>::SMEM_BYTES, stream, mq, mk, mv, (__nv_bfloat16*)out, o_stride,
              block_table, max_pages, seq_slot, cu_q, kv_len, nq, nkv, scale, window, heads_first, strict_order, status);
    return RB_OK;
}
}  // namespace

// q rows [T, q_stride] bfloat16 (T = tokens of the step), caches [n_pages, nkv, 64, hd].  heads_first: the order
// in which blocks start (see the kernel); it changes no result.  Head sizes 64, 128 and 256;
// RB_ERR_BAD_SIZE / RB_ERR_BAD_ALIGN otherwise (the caller then uses the mma.sync kernel).
extern "C" int rb_attention_prefill_tc5(const void* q, int q_stride, int T, void* out, int o_stride,
                                        const void* k_cache, const void* v_cache, int n_pages,
                                        const int* block_table, int max_pages, const int* seq_slot,
                                        const int* cu_q, const int* kv_len, int B, int max_q_len, int nq, int nkv,
                                        int hd, float scale, int window, int heads_first, int* status, void* stream) {
    if (B <= 0 || max_q_len <= 0 || T <= 0) return RB_OK;
    if ((hd != 64 && hd != 128 && hd != 256) || nkv <= 0 || nq % nkv) return RB_ERR_BAD_SIZE;
    if (((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15) || ((uintptr_t)out & 15) ||
        (q_stride % 8) || (o_stride % 8))
        return RB_ERR_BAD_ALIGN;
#define RB_TC5_ARGS q, q_stride, T, out, o_stride, k_cache, v_cache, n_pages, block_table, max_pages, seq_slot, cu_q, kv_len, \
                    B, max_q_len, nq, nkv, scale, window, heads_first, status, (cudaStream_t)stream
    if (hd == 64) return launch_tc5<64>(RB_TC5_ARGS);
    if (hd == 128) return launch_tc5<128>(RB_TC5_ARGS);
    return launch_tc5<256>(RB_TC5_ARGS);
#undef RB_TC5_ARGS
}
