// bfloat16 matrix product on the 5th-generation tensor cores:
//     out[M, N] = x[M, K] . W[N, K]^T (+ bias), float32 accumulation in tensor memory.
//
// Both operands are K-major, so one kernel serves both shapes of the engine by choosing which
// operand sits on the 128-row side of the MMA:
//   * many tokens (prefill):  A = x (128 tokens per tile),   B = W (BN features per tile)
//   * few tokens  (decode):   A = W (128 features per tile), B = x (BN >= tokens, 16..128)
//     so that the weights, which are all the traffic, stream through full-height MMAs while
//     the handful of tokens sits on the N side; the tile is written back transposed.
// Per CTA: warp 0 issues TMA loads into a ring of shared-memory stages (128-byte swizzle),
// warp 1 allocates tensor memory and issues tcgen05.mma (one elected thread), warps 2-5 read
// the accumulator with tcgen05.ld and store.  K can be split over blockIdx.z; each split
// writes its own float32 partial result (the consumer sums them in a fixed order).
//
// It stands where the reference has gemv_f16 (decode) and gemm_xwt_f16 (prefill):
// rocml-kernels/kernels/gemv_f16.hip:8-36, gemm_f16.hip:10-41.
#include <type_traits>
#include "common.cuh"
#include "sm100.cuh"
#include "api.h"
#include <cstdlib>
#include <mutex>
#include <unordered_map>

using namespace sm100;

namespace {

constexpr int BM = 128;      // rows of the A operand per tile (UMMA M)
constexpr int BK = 64;       // bf16 elements per stage row: 128 bytes, one swizzle atom
constexpr int UMMA_K = 16;
constexpr int SMEM_BUDGET = 200 * 1024;

template <int BN>
struct Cfg {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int B_STRIDE = (B_BYTES + 1023) / 1024 * 1024;  // keep every stage 1024-aligned
    static constexpr int STAGE = A_BYTES + B_STRIDE;
    static constexpr int STAGES_RAW = SMEM_BUDGET / STAGE;
    static constexpr int STAGES = STAGES_RAW > 10 ? 10 : STAGES_RAW;
    static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
    static constexpr int SMEM = STAGES * STAGE + 1024 /*align slack*/ + 256 /*barriers*/;   // the persistent kernel's
};

struct Params {
    int a_rows, b_rows, K;        // extents of the A-side and B-side operands
    int splits;                   // the K blocks are dealt out evenly over blockIdx.z
    long long ldo;                // row stride of out, in elements
    long long split_stride;       // elements between the partial results of two splits
    const float* bias;            // [features] or null; added by split 0 only
    int* status;
    int stages;                   // depth of the shared-memory ring actually used (<= Cfg::STAGES)
    long long wait_cycles;        // after this many clock cycles a wait on a barrier gives up
    int withhold;                 // tests only: the first stage's copies are never issued, so its barrier never completes
    // CS >= 4 (the product is added into the residual stream, see the kernel):
    float* resid;                 // [tokens][features] float32, updated in place
    long long resid_ld;
    const void* next_w;           // the following norm's weight [features], or null
    int next_w_f32;               // its type: float32 or bfloat16
    __nv_bfloat16* xhat;          // [tokens][features]: resid * next_w, not yet divided by the row's RMS
    long long xhat_ld;
    float* sumsq;                 // [feature groups][tokens]: sums of squares of the new residual rows
    long long sumsq_ld;
    // CS == 2: the input rows still lack the norm's 1/RMS; it is applied to the product instead
    const float* row_sumsq;       // [row_groups][tokens] shares of the input rows' sums of squares, or null
    int row_groups;
    long long row_sumsq_ld;
    float row_eps, row_inv_width; // 1/RMS = rsqrt(sum * row_inv_width + row_eps)
    // pair kernel, EPI == 2: the product is a prompt's q | k | v projection with heads of 128
    __nv_bfloat16* q_out;         // [tokens][nq * 128], row stride q_ld
    long long q_ld;
    __nv_bfloat16* k_cache;       // [pages][nkv][64][128]
    __nv_bfloat16* v_cache;
    const int* positions;         // per token
    const int* slot_of_token;     // per token, < 0: padding
    const int* block_table;       // [slots][max_pages]
    int max_pages;
    const void* q_norm_w;         // [128] or null
    const void* k_norm_w;
    int norm_w_f32;
    float norm_eps;
    const float2* cos_sin;        // [tokens][64] (cos, sin), or null
    int nq, nkv;
};

// 16 consecutive outputs as 16-byte stores (dst is 16-byte aligned).
__device__ __forceinline__ void store16(float* dst, const float* v) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
        reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
}
__device__ __forceinline__ void load16(const float* src, float* v) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 f = reinterpret_cast<const float4*>(src)[i];
        v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
    }
}
__device__ __forceinline__ void store16(__nv_bfloat16* dst, const float* v) {
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    reinterpret_cast<uint4*>(dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
    reinterpret_cast<uint4*>(dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
}

// CS = 2 (few tokens, a gate/up weight, the sum over K in two halves): the two blocks of a tile are
// a thread-block cluster.  The second half's block hands its accumulator to the first through
// distributed shared memory, and the first adds it to its own and writes silu(gate) * up: no
// partial sums go through global memory and no second kernel has to wait for them.
// CS = 4, 8 or 16 (few tokens, a product that is added to the residual stream, the sum over K in CS
// parts): the CS blocks of a tile are a cluster.  Each block owns 128 / CS of the tile's features;
// every block sends each owner its part of them through distributed shared memory, and after one
// cluster barrier the owner adds the parts in order, adds the bias and the residual, writes the new
// residual (float32), and for the norm that follows: residual * weight in bfloat16 (the next product's
// input, to be scaled by the row's 1/RMS in that product's epilogue) and its share of the row's sum
// of squares.  No partial sums go through global memory and no norm kernel runs in between.
template <int BN, bool SWAP, typename OT, bool GATED, int CS>
__global__ void __launch_bounds__(192, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    OT* __restrict__ out, const Params p) {
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int S = p.stages;
    uint64_t* full = (uint64_t*)(smem + S * C::STAGE);
    uint64_t* empty = full + S;
    uint64_t* acc_ready = empty + S;
    uint32_t* tmem_slot = (uint32_t*)(acc_ready + 1);
    uint32_t* abort_flag = tmem_slot + 1;
    float* handover = (float*)(smem + S * C::STAGE + 256);   // CS: [BN][128] floats from the other half
    __shared__ float s_rstd[CS == 2 ? BN : 1];               // CS == 2: the tokens' 1/RMS

    rb::pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int a0 = blockIdx.x * BM;   // first row of the A-side operand in this tile
    const int b0 = blockIdx.y * BN;   // first row of the B-side operand
    const int kb_total = (p.K + BK - 1) / BK;
    const int kb_first = (int)((long long)blockIdx.z * kb_total / p.splits);
    const int n_kb = (int)((long long)(blockIdx.z + 1) * kb_total / p.splits) - kb_first;
    const int k_begin = kb_first * BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(acc_ready, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    int issued = 0;                   // K blocks whose copies the producer thread has requested
    if (warp == 0) {
        if (lane == 0) {
            tma_prefetch_desc(&map_a);
            tma_prefetch_desc(&map_b);
            // The weights do not depend on the kernel before this one: their first tiles are
            // requested at once, then the predecessor's results are waited for, then the
            // activations' tiles follow.
            const int pre = n_kb < S ? n_kb : S;
            // p.withhold (tests only): nothing is requested for the first stage, so nothing is in flight
            // for it and its barrier never completes: the warp that waits for it must give up
            const int kb0 = (CS == 0 && p.withhold) ? 1 : 0;      // only the plain kernel honours the switch
            for (int kb = kb0; kb < pre; ++kb) {
                uint8_t* sa = smem + kb * C::STAGE;
                mbar_arrive_expect_tx(&full[kb], C::A_BYTES + C::B_BYTES);
                if (SWAP) tma_load_2d(sa, &map_a, k_begin + kb * BK, a0, &full[kb]);
                else tma_load_2d(sa + C::A_BYTES, &map_b, k_begin + kb * BK, b0, &full[kb]);
            }
            rb::pdl_wait();
            for (int kb = kb0; kb < pre; ++kb) {
                uint8_t* sa = smem + kb * C::STAGE;
                if (SWAP) tma_load_2d(sa + C::A_BYTES, &map_b, k_begin + kb * BK, b0, &full[kb]);
                else tma_load_2d(sa, &map_a, k_begin + kb * BK, a0, &full[kb]);
            }
            issued = pre;
            bool ok = true;
            // a lone thread executes a dependent instruction every few cycles at best: the stage, its parity and
            // the K coordinate are carried along instead of being divided out of kb every time
            int s = pre == S ? 0 : pre;
            uint32_t par = 0;                 // the parity to wait for on empty[s]: the first refill waits for use 0
            int c0 = k_begin + pre * BK;
            for (int kb = pre; kb < n_kb; ++kb) {
                if (!mbar_try_wait(&empty[s], par)) {
                    ok = mbar_wait(&empty[s], par, p.wait_cycles);
                    if (!ok) break;
                }
                uint8_t* sa = smem + s * C::STAGE;
                mbar_arrive_expect_tx(&full[s], C::A_BYTES + C::B_BYTES);
                tma_load_2d(sa, &map_a, c0, a0, &full[s]);
                tma_load_2d(sa + C::A_BYTES, &map_b, c0, b0, &full[s]);
                ++issued;
                c0 += BK;
                if (++s == S) { s = 0; par ^= 1u; }
            }
            if (!ok) {
                atomicExch(p.status, RB_ERR_TIMEOUT);
                atomicExch(abort_flag, 1u);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_bf16_f32(BM, BN);
            bool ok = true;
            const uint32_t a_lo0 = smem_desc_sw128_lo(smem_u32(smem));
            uint32_t a_lo = a_lo0, par = 0;
            int s = 0;
            for (int kb = 0; kb < n_kb; ++kb) {
                if (!mbar_try_wait(&full[s], par)) {
                    ok = mbar_wait(&full[s], par, p.wait_cycles);
                    if (!ok) break;
                }
                tc_fence_after();
                mma_bf16_k64(tmem_base, a_lo, a_lo + (C::A_BYTES >> 4), idesc, kb == 0 ? 1u : 0u);
                mma_commit(&empty[s]);   // the stage is free once these MMAs have read it
                a_lo += C::STAGE >> 4;
                if (++s == S) { s = 0; par ^= 1u; a_lo = a_lo0; }
            }
            if (!ok) {
                atomicExch(p.status, RB_ERR_TIMEOUT);
                atomicExch(abort_flag, 1u);
            }
            mma_commit(acc_ready);       // completes when everything issued has finished
        }
    } else {
        // epilogue warps 2..5: warp w may read TMEM lanes 32 * (w % 4) .. + 31
        const int quarter = warp & 3;
        const bool ok = __all_sync(0xffffffffu, mbar_wait(acc_ready, 0, p.wait_cycles));  // warp-uniform
        tc_fence_after();
        const bool aborted = !ok || *(volatile uint32_t*)abort_flag != 0;
        if (!ok && lane == 0) atomicExch(p.status, RB_ERR_TIMEOUT);
        if (CS >= 4) {
            // every block sends each owner its rows of the accumulator
            if (!aborted && n_kb > 0) {
                constexpr int RPC = 128 / (CS >= 4 ? CS : 4);       // features a block owns
                const int row = quarter * 32 + lane;
                const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
                const uint32_t dst = map_to_cta(smem_u32(handover + (size_t)blockIdx.z * BN * RPC + row % RPC), row / RPC);
#pragma unroll 1
                for (int c = 0; c < BN / 16; ++c) {
                    float v[16];
                    tmem_ld16(lane_addr + c * 16, v);
#pragma unroll
                    for (int i = 0; i < 16; ++i) st_cluster_f32(dst + (uint32_t)((c * 16 + i) * RPC * 4), v[i]);
                }
            }
        } else if (CS != 0) {
            // the second half hands its accumulator over; the first half goes on after the barrier
            if (blockIdx.z == 0 && p.row_sumsq != nullptr) {
                // meanwhile: the 1/RMS of this tile's tokens, from the shares the kernel before left
                rb::pdl_wait();
                for (int j = quarter; j < BN; j += 4) {
                    const int tok = b0 + j;
                    float acc = 0.f;
                    if (tok < p.b_rows)
                        for (int gi = lane; gi < p.row_groups; gi += 32) acc += p.row_sumsq[(size_t)gi * p.row_sumsq_ld + tok];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                    if (lane == 0) s_rstd[j] = rsqrtf(acc * p.row_inv_width + p.row_eps);
                }
            }
            if (!aborted && n_kb > 0 && blockIdx.z != 0) {
                const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
                const uint32_t dst = map_to_cta(smem_u32(handover + quarter * 32 + lane), 0);
#pragma unroll 1
                for (int c = 0; c < BN / 16; ++c) {
                    float v[16];
                    tmem_ld16(lane_addr + c * 16, v);
#pragma unroll
                    for (int i = 0; i < 16; ++i) st_cluster_f32(dst + (uint32_t)((c * 16 + i) * 128 * 4), v[i]);
                }
            }
        } else if (!aborted && n_kb > 0) {
            const int ar = a0 + quarter * 32 + lane;   // this thread's row of the A-side operand
            OT* o = out + (size_t)blockIdx.z * p.split_stride;
            const bool add_bias = p.bias != nullptr && blockIdx.z == 0;
            const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
            const bool vec_ok = (((uintptr_t)o | ((uintptr_t)p.ldo * sizeof(OT))) & 15) == 0;
            if (GATED) {
                // The weight's rows alternate in blocks of 16 between the gate and the up projection
                // of the same 16 outputs; the tile's value is silu(gate) * up (silu(g) = g / (1 + exp(-g)),
                // rocml-kernels/kernels/silu_mul.hip:15-18), half as wide as the product.
                if (SWAP) {
                    // features on the TMEM lanes: lanes 0-15 of a warp hold gates, lanes 16-31 the ups
                    const float bv = (add_bias && ar < p.a_rows) ? p.bias[ar] : 0.f;
                    const int fo = (ar >> 5) * 16 + (lane & 15);
#pragma unroll 1
                    for (int c = 0; c < BN / 16; ++c) {
                        float v[16];
                        tmem_ld16(lane_addr + c * 16, v);
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const float mine = v[i] + bv;
                            const float up = __shfl_down_sync(0xffffffffu, mine, 16);
                            const int tok = b0 + c * 16 + i;
                            if (lane < 16 && tok < p.b_rows && ar < p.a_rows)
                                o[(size_t)tok * p.ldo + fo] = rb::from_f32<OT>(mine / (1.f + expf(-mine)) * up);
                        }
                    }
                } else {
                    OT* row = o + (size_t)(ar < p.a_rows ? ar : 0) * p.ldo;
#pragma unroll 1
                    for (int c = 0; c < BN / 16; c += 2) {
                        float g[16], u[16];
                        tmem_ld16(lane_addr + c * 16, g);
                        tmem_ld16(lane_addr + (c + 1) * 16, u);
                        const int f0 = b0 + c * 16;                 // gate columns f0.., up columns f0 + 16..
                        if (ar < p.a_rows && f0 + 32 <= p.b_rows) {
                            if (add_bias) {
#pragma unroll
                                for (int i = 0; i < 16; ++i) { g[i] += p.bias[f0 + i]; u[i] += p.bias[f0 + 16 + i]; }
                            }
#pragma unroll
                            for (int i = 0; i < 16; ++i) g[i] = g[i] / (1.f + expf(-g[i])) * u[i];
                            OT* dst = row + (f0 >> 1);
                            if (vec_ok) store16(dst, g);
                            else {
#pragma unroll
                                for (int i = 0; i < 16; ++i) dst[i] = rb::from_f32<OT>(g[i]);
                            }
                        }
                    }
                }
            } else
#pragma unroll 1
            for (int c = 0; c < BN / 16; ++c) {
                float v[16];
                tmem_ld16(lane_addr + c * 16, v);
                if (SWAP) {

                    // A side = features, B side = tokens: out[token][feature]
                    const float bv = (add_bias && ar < p.a_rows) ? p.bias[ar] : 0.f;
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int tok = b0 + c * 16 + i;
                        if (tok < p.b_rows && ar < p.a_rows)
                            o[(size_t)tok * p.ldo + ar] = rb::from_f32<OT>(v[i] + bv);
                    }
                } else {
                    // A side = tokens, B side = features: out[token][feature]; this thread owns 16
                    // consecutive features of its row: 32 or 64 contiguous bytes, written as 16-byte
                    // stores when the row is aligned and the chunk lies inside the matrix
                    if (ar < p.a_rows) {
                        OT* row = o + (size_t)ar * p.ldo;
                        const int f0 = b0 + c * 16;
                        if (add_bias) {
#pragma unroll
                            for (int i = 0; i < 16; ++i) v[i] += (f0 + i < p.b_rows) ? p.bias[f0 + i] : 0.f;
                        }
                        if (vec_ok && f0 + 16 <= p.b_rows) {
                            store16(row + f0, v);
                        } else {
#pragma unroll
                            for (int i = 0; i < 16; ++i)
                                if (f0 + i < p.b_rows) row[f0 + i] = rb::from_f32<OT>(v[i]);
                        }
                    }
                }
            }
        }
    }
    if (CS != 0) {
        // every thread of both blocks, whatever happened to it above
        // what the first round below reads from global memory is requested before the barrier, so that it
        // arrives while the blocks wait for one another (a block is the only writer of its residual rows)
        float first_r = 0.f, first_w = 1.f, first_b = 0.f;
        if (CS >= 4 && warp >= 2) {
            rb::pdl_wait();   // these threads read what earlier kernels wrote (the residual): returns at once by now
            constexpr int RPC = 128 / (CS >= 4 ? CS : 4);
            const int e = (warp & 3) * 32 + lane;
            const int tok = b0 + e / RPC, n = a0 + (int)blockIdx.z * RPC + e % RPC;
            if (e < RPC * BN && tok < p.b_rows && n < p.a_rows) {
                first_r = p.resid[(size_t)tok * p.resid_ld + n];
                if (p.bias != nullptr) first_b = p.bias[n];
                if (p.xhat != nullptr)
                    first_w = p.next_w_f32 ? static_cast<const float*>(p.next_w)[n]
                                           : __bfloat162float(static_cast<const __nv_bfloat16*>(p.next_w)[n]);
            }
        }
        __syncwarp();
        cluster_arrive();
        cluster_wait();
        if (CS >= 4 && warp >= 2) {
            constexpr int RPC = 128 / (CS >= 4 ? CS : 4);
            const int e = (warp & 3) * 32 + lane;                   // 0..127 among the epilogue threads
#pragma unroll 1
            for (int idx = e; idx < RPC * BN; idx += 128) {
                const int row_in = idx % RPC, tok = b0 + idx / RPC;
                const int n = a0 + (int)blockIdx.z * RPC + row_in;
                const bool valid = tok < p.b_rows && n < p.a_rows;
                float val = 0.f;
#pragma unroll
                for (int src = 0; src < CS; ++src) val += handover[((size_t)src * BN + idx / RPC) * RPC + row_in];
                float sq = 0.f;
                if (valid) {
                    float* rp = p.resid + (size_t)tok * p.resid_ld + n;
                    const bool pre = idx == e;                      // the first round's values are here already
                    const float r_new = (pre ? first_r : *rp) + val + (pre ? first_b : (p.bias != nullptr ? p.bias[n] : 0.f));
                    *rp = r_new;
                    sq = r_new * r_new;
                    if (p.xhat != nullptr) {
                        const float wn = pre ? first_w
                                             : (p.next_w_f32 ? static_cast<const float*>(p.next_w)[n]
                                                             : __bfloat162float(static_cast<const __nv_bfloat16*>(p.next_w)[n]));
                        p.xhat[(size_t)tok * p.xhat_ld + n] = __float2bfloat16_rn(r_new * wn);
                    }
                }
#pragma unroll
                for (int o = RPC / 2; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
                if (row_in == 0 && tok < p.b_rows && p.sumsq != nullptr)
                    p.sumsq[((size_t)blockIdx.x * CS + blockIdx.z) * p.sumsq_ld + tok] = sq;
            }
        } else if (blockIdx.z == 0 && warp >= 2 && n_kb > 0 && *(volatile uint32_t*)abort_flag == 0) {
            // features on the TMEM lanes: lanes 0-15 of a warp hold gates, lanes 16-31 the ups
            const int quarter = warp & 3;
            const int ar = a0 + quarter * 32 + lane;
            const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
            const float bv = (p.bias != nullptr && ar < p.a_rows) ? p.bias[ar] : 0.f;
            const int fo = (ar >> 5) * 16 + (lane & 15);
            const float* other = handover + quarter * 32 + lane;
            tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < BN / 16; ++c) {
                float v[16];
                tmem_ld16(lane_addr + c * 16, v);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float rs = p.row_sumsq != nullptr ? s_rstd[c * 16 + i] : 1.f;
                    const float mine = (v[i] + other[(c * 16 + i) * 128]) * rs + bv;   // first half + second half
                    const float up = __shfl_down_sync(0xffffffffu, mine, 16);
                    const int tok = b0 + c * 16 + i;
                    if (lane < 16 && tok < p.b_rows && ar < p.a_rows)
                        out[(size_t)tok * p.ldo + fo] = rb::from_f32<OT>(mine / (1.f + expf(-mine)) * up);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0 && lane == 0 && *(volatile uint32_t*)abort_flag != 0) {
        // Somebody gave up.  Before the block leaves, the producer waits (bounded) for the copies it
        // still has in flight into this block's shared memory: the last S it requested.
        const int first = issued > S ? issued - S : 0;
        for (int kb = first; kb < issued; ++kb)
            if (!(CS == 0 && p.withhold && kb == 0)) mbar_wait(&full[kb % S], (kb / S) & 1, p.wait_cycles);
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}


// ---- many tokens: a persistent kernel with two accumulators ---------------------------------------
// One block per multiprocessor walks over the output tiles (tokens on the 128-row side, BN features
// per tile; tiles that share a weight tile are neighbours, so the weight is read from memory once).
// Tensor memory holds TWO accumulators of BN columns: while the 4 epilogue warps read tile i out of
// one (bias, the gated activation, conversion, 16-byte stores), the MMA warp already fills the other
// with tile i + 1, and the TMA warp runs ahead through the same shared-memory ring across tile
// boundaries.  The epilogue thus costs nothing as long as it is shorter than a tile's main loop.
template <int BN, typename OT, bool GATED>
__global__ void __launch_bounds__(192, 1)
gemm_tcgen05_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                               OT* __restrict__ out, const Params p) {
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int S = p.stages;
    uint64_t* full = (uint64_t*)(smem + S * C::STAGE);
    uint64_t* empty = full + S;
    uint64_t* acc_full = empty + S;      // [2]
    uint64_t* acc_empty = acc_full + 2;  // [2]
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    uint32_t* abort_flag = tmem_slot + 1;

    rb::pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_tiles = (p.a_rows + BM - 1) / BM, n_tiles = (p.b_rows + BN - 1) / BN;
    const int n_total = m_tiles * n_tiles;
    const int n_kb = (p.K + BK - 1) / BK;
    constexpr int TMEM_COLS = 2 * C::TMEM_COLS;   // 512 at BN = 256

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 4); }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            tma_prefetch_desc(&map_a);
            tma_prefetch_desc(&map_b);
            long long it = 0;          // K blocks issued so far, over all tiles: the ring's position
            bool ok = true, waited = false;
            for (int tile = blockIdx.x; tile < n_total && ok; tile += gridDim.x) {
                const int a0 = (tile % m_tiles) * BM, b0 = (tile / m_tiles) * BN;
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = (int)(it % S);
                    const uint32_t ph = (uint32_t)((it / S) & 1);
                    ok = mbar_wait(&empty[s], ph ^ 1, p.wait_cycles);
                    if (!ok) break;
                    uint8_t* sa = smem + s * C::STAGE;
                    mbar_arrive_expect_tx(&full[s], C::A_BYTES + C::B_BYTES);
                    tma_load_2d(sa + C::A_BYTES, &map_b, kb * BK, b0, &full[s]);    // weights: independent
                    if (!waited && (it + 1 == S || (tile + gridDim.x >= n_total && kb + 1 == n_kb))) {
                        // the ring is primed with weight tiles: now wait for the predecessor's
                        // results, then send the activations' tiles of everything issued so far
                        rb::pdl_wait();
                        waited = true;
                        for (long long j = 0; j <= it; ++j) {
                            const int tj = blockIdx.x + (int)(j / n_kb) * gridDim.x;
                            tma_load_2d(smem + (int)(j % S) * C::STAGE, &map_a, (int)(j % n_kb) * BK,
                                        (tj % m_tiles) * BM, &full[(int)(j % S)]);
                        }
                    } else if (waited) {
                        tma_load_2d(sa, &map_a, kb * BK, a0, &full[s]);
                    }
                }
            }
            if (!waited) rb::pdl_wait();
            if (!ok) {
                atomicExch(p.status, RB_ERR_TIMEOUT);
                atomicExch(abort_flag, 1u);
                const long long first = it > S ? it - S : 0;
                for (long long j = first; j < it; ++j) mbar_wait(&full[(int)(j % S)], (uint32_t)((j / S) & 1), p.wait_cycles);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_bf16_f32(BM, BN);
            long long it = 0;
            int local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_total && ok; tile += gridDim.x, ++local) {
                const int acc = local & 1;
                const uint32_t use = (uint32_t)(local >> 1);
                ok = mbar_wait(&acc_empty[acc], (use & 1) ^ 1, p.wait_cycles);    // the epilogue has drained this accumulator
                if (!ok) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + acc * C::TMEM_COLS;
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = (int)(it % S);
                    ok = mbar_wait(&full[s], (uint32_t)((it / S) & 1), p.wait_cycles);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + s * C::STAGE);
                    const uint64_t adesc = smem_desc_sw128(sa);
                    const uint64_t bdesc = smem_desc_sw128(sa + C::A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        mma_bf16(tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    mma_commit(&empty[s]);
                }
                if (!ok) break;
                mma_commit(&acc_full[acc]);
            }
            if (!ok) {
                atomicExch(p.status, RB_ERR_TIMEOUT);
                atomicExch(abort_flag, 1u);
                mma_commit(&acc_full[0]);     // wake the epilogue, which then sees the abort flag
                mma_commit(&acc_full[1]);
            }
        }
    } else {
        const int quarter = warp & 3;
        int local = 0;
        for (int tile = blockIdx.x; tile < n_total; tile += gridDim.x, ++local) {
            const int acc = local & 1;
            const uint32_t use = (uint32_t)(local >> 1);
            const bool ok = __all_sync(0xffffffffu, mbar_wait(&acc_full[acc], use & 1, p.wait_cycles));
            tc_fence_after();
            if (!ok || *(volatile uint32_t*)abort_flag != 0) {
                if (!ok && lane == 0) atomicExch(p.status, RB_ERR_TIMEOUT);
                break;
            }
            const int a0 = (tile % m_tiles) * BM, b0 = (tile / m_tiles) * BN;
            const int ar = a0 + quarter * 32 + lane;
            const bool add_bias = p.bias != nullptr;
            const uint32_t lane_addr = tmem_base + acc * C::TMEM_COLS + ((uint32_t)(quarter * 32) << 16);
            const bool vec_ok = (((uintptr_t)out | ((uintptr_t)p.ldo * sizeof(OT))) & 15) == 0;
            OT* row = out + (size_t)(ar < p.a_rows ? ar : 0) * p.ldo;
            if (GATED) {
#pragma unroll 1
                for (int c = 0; c < BN / 16; c += 2) {
                    float g[16], u[16];
                    tmem_ld16(lane_addr + c * 16, g);
                    tmem_ld16(lane_addr + (c + 1) * 16, u);
                    const int f0 = b0 + c * 16;
                    if (ar < p.a_rows && f0 + 32 <= p.b_rows) {
                        if (add_bias) {
#pragma unroll
                            for (int i = 0; i < 16; ++i) { g[i] += p.bias[f0 + i]; u[i] += p.bias[f0 + 16 + i]; }
                        }
#pragma unroll
                        for (int i = 0; i < 16; ++i) g[i] = g[i] / (1.f + expf(-g[i])) * u[i];
                        OT* dst = row + (f0 >> 1);
                        if (vec_ok) store16(dst, g);
                        else {
#pragma unroll
                            for (int i = 0; i < 16; ++i) dst[i] = rb::from_f32<OT>(g[i]);
                        }
                    }
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < BN / 16; ++c) {
                    float v[16];
                    tmem_ld16(lane_addr + c * 16, v);
                    const int f0 = b0 + c * 16;
                    if (ar < p.a_rows) {
                        if (add_bias) {
#pragma unroll
                            for (int i = 0; i < 16; ++i) v[i] += (f0 + i < p.b_rows) ? p.bias[f0 + i] : 0.f;
                        }
                        if (vec_ok && f0 + 16 <= p.b_rows) {
                            store16(row + f0, v);
                        } else {
#pragma unroll
                            for (int i = 0; i < 16; ++i)
                                if (f0 + i < p.b_rows) row[f0 + i] = rb::from_f32<OT>(v[i]);
                        }
                    }
                }
            }
            // this warp has read all it needs of the accumulator: hand it back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[acc]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}


// ---- many tokens, pairs of CTAs (cta_group::2) -------------------------------------------------------
// Two CTAs of a cluster compute a 256 x 256 output tile together: each loads its own 128 rows of the
// tokens and its own HALF (128 rows) of the weight tile, the even CTA's MMA warp issues
// tcgen05.mma.cta_group::2 (M = 256), which reads both CTAs' shared memory and writes each CTA's 128
// rows of the accumulator into that CTA's tensor memory.  Per multiprocessor this halves the bytes
// of the weight operand that are loaded and read from shared memory per MMA, which is what bounds
// the single-CTA kernel (128 x 256 tiles read 96 bytes per clock of a 128-byte-per-clock port).
// Persistent, two accumulators, as the single-CTA kernel above.  Barriers: full[] is counted on the
// leader (both CTAs' TMA loads report there), empty[] and acc_full[] exist in both CTAs and are
// signalled by multicast commits, acc_empty[] lives in the leader and collects the 8 epilogue warps
// of the pair.  No TMA multicast is used anywhere.
constexpr int PAIR_BN = 256;
constexpr int PAIR_STAGE = 2 * BM * BK * 2;       // A 128 x 64 + B half 128 x 64, bf16: 32 KB
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_SMEM = PAIR_STAGES * PAIR_STAGE + 1024 + 256;

// EPI: 0 plain, 3 added into `out` (the float32 residual stream) instead of written, 1 SiLU(gate) * up (rows
// of the weight interleaved by 16), 2 a prompt's q | k | v projection
// with heads of 128: a tile's 256 columns are two whole heads and an epilogue thread owns a token, so
// the per-head RMSNorm and the rotation (pairs i, i + 64) are done on the accumulator itself, and
// the queries go to their own tensor, keys and values straight into their cache pages.
template <typename OT, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         OT* __restrict__ out, const Params p) {
    constexpr int BN = PAIR_BN, S = PAIR_STAGES, A_BYTES = BM * BK * 2;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(smem + S * PAIR_STAGE);
    uint64_t* empty = full + S;
    uint64_t* acc_full = empty + S;      // [2]
    uint64_t* acc_empty = acc_full + 2;  // [2], used in the leader
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    uint32_t* abort_flag = tmem_slot + 1;

    rb::pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int m_pairs = (p.a_rows + 2 * BM - 1) / (2 * BM), n_tiles = (p.b_rows + BN - 1) / BN;
    const int n_total = m_pairs * n_tiles;
    const int n_kb = (p.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 8); }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, 512);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_arrive();           // the peer's barriers are initialised before anything signals them
    cluster_wait();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            tma_prefetch_desc(&map_a);
            tma_prefetch_desc(&map_b);
            rb::pdl_wait();
            long long it = 0;
            bool ok = true;
            for (int tile = pair; tile < n_total && ok; tile += n_pairs) {
                const int a0 = (tile % m_pairs) * 2 * BM + (int)rank * BM;
                const int b0 = (tile / m_pairs) * BN + (int)rank * (BN / 2);
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = (int)(it % S);
                    ok = mbar_wait(&empty[s], (uint32_t)(((it / S) & 1) ^ 1), p.wait_cycles);
                    if (!ok) break;
                    uint8_t* sa = smem + s * PAIR_STAGE;
                    const uint32_t bar = smem_u32(&full[s]) & PEER_BIT_MASK;   // the leader's barrier
                    if (rank == 0) mbar_arrive_expect_tx(&full[s], 2 * PAIR_STAGE);   // both CTAs' bytes
                    tma_load_2d_pair(sa + A_BYTES, &map_b, kb * BK, b0, bar);
                    tma_load_2d_pair(sa, &map_a, kb * BK, a0, bar);
                }
            }
            if (!ok) {
                atomicExch(p.status, RB_ERR_TIMEOUT);
                atomicExch(abort_flag, 1u);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = idesc_bf16_f32(2 * BM, BN);
            long long it = 0;
            int local = 0;
            bool ok = true;
            for (int tile = pair; tile < n_total && ok; tile += n_pairs, ++local) {
                const int acc = local & 1;
                const uint32_t use = (uint32_t)(local >> 1);
                ok = mbar_wait(&acc_empty[acc], (use & 1) ^ 1, p.wait_cycles);
                if (!ok) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + acc * BN;
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = (int)(it % S);
                    ok = mbar_wait(&full[s], (uint32_t)((it / S) & 1), p.wait_cycles);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + s * PAIR_STAGE);
                    const uint64_t adesc = smem_desc_sw128(sa);
                    const uint64_t bdesc = smem_desc_sw128(sa + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        mma_bf16_pair(tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    mma_commit_pair(&empty[s]);          // frees the stage in both CTAs
                }
                if (!ok) break;
                mma_commit_pair(&acc_full[acc]);         // wakes both CTAs' epilogue warps
            }
            if (!ok) {
                atomicExch(p.status, RB_ERR_TIMEOUT);
                atomicExch(abort_flag, 1u);
                mma_commit_pair(&acc_full[0]);
                mma_commit_pair(&acc_full[1]);
            }
        }
    } else {
        const int quarter = warp & 3;
        int local = 0;
        for (int tile = pair; tile < n_total; tile += n_pairs, ++local) {
            const int acc = local & 1;
            const uint32_t use = (uint32_t)(local >> 1);
            const bool ok = __all_sync(0xffffffffu, mbar_wait(&acc_full[acc], use & 1, p.wait_cycles));
            tc_fence_after();
            if (!ok || *(volatile uint32_t*)abort_flag != 0) {
                if (!ok && lane == 0) atomicExch(p.status, RB_ERR_TIMEOUT);
                break;
            }
            const int a0 = (tile % m_pairs) * 2 * BM + (int)rank * BM, b0 = (tile / m_pairs) * BN;
            const int ar = a0 + quarter * 32 + lane;
            const bool add_bias = p.bias != nullptr;
            const uint32_t lane_addr = tmem_base + acc * BN + ((uint32_t)(quarter * 32) << 16);
            const bool vec_ok = (((uintptr_t)out | ((uintptr_t)p.ldo * sizeof(OT))) & 15) == 0;
            OT* row = out + (size_t)(ar < p.a_rows ? ar : 0) * p.ldo;
            if (EPI == 2) {
                rb::pdl_wait();   // these threads read what an earlier kernel wrote (the angles' table): returns at once by now
                int slot = -1, pos = 0, page = -2;         // page -2: not looked up yet
                if (ar < p.a_rows) { slot = p.slot_of_token[ar]; pos = p.positions[ar]; }
#pragma unroll 1
                for (int hh = 0; hh < BN / 128; ++hh) {
                    const int col0 = b0 + hh * 128;
                    if (col0 >= p.b_rows) break;
                    const int head = col0 >> 7;
                    const int kind = head < p.nq ? 0 : (head < p.nq + p.nkv ? 1 : 2);
                    __nv_bfloat16* dst = nullptr;
                    if (slot >= 0) {
                        if (kind == 0) {
                            dst = p.q_out + (size_t)ar * p.q_ld + (size_t)head * 128;
                        } else {
                            if (page == -2) page = p.block_table[(size_t)slot * p.max_pages + (pos / RB_PAGE)];
                            const int hk = kind == 1 ? head - p.nq : head - p.nq - p.nkv;
                            if (page >= 0)
                                dst = (kind == 1 ? p.k_cache : p.v_cache) +
                                      (((size_t)page * p.nkv + hk) * RB_PAGE + (pos % RB_PAGE)) * 128;
                        }
                    }
                    const uint32_t hbase = lane_addr + hh * 128;
                    const void* w = kind == 0 ? p.q_norm_w : (kind == 1 ? p.k_norm_w : nullptr);
                    float inv = 1.f;
                    if (w != nullptr) {
                        float ss = 0.f;
#pragma unroll 1
                        for (int c = 0; c < 8; ++c) {
                            float v[16];
                            tmem_ld16(hbase + c * 16, v);
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                const float x = v[i] + (add_bias ? p.bias[col0 + c * 16 + i] : 0.f);
                                ss += x * x;
                            }
                        }
                        inv = rsqrtf(ss / 128.f + p.norm_eps);
                    }
                    const bool rotate = kind != 2 && p.cos_sin != nullptr;
#pragma unroll 1
                    for (int c = 0; c < 4; ++c) {
                        float lo[16], hi[16];
                        tmem_ld16(hbase + c * 16, lo);
                        tmem_ld16(hbase + (c + 4) * 16, hi);
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const int d = c * 16 + i;
                            float a = lo[i], b = hi[i];
                            if (add_bias) { a += p.bias[col0 + d]; b += p.bias[col0 + 64 + d]; }
                            if (w != nullptr) {
                                const float wa = p.norm_w_f32 ? static_cast<const float*>(w)[d]
                                                              : __bfloat162float(static_cast<const __nv_bfloat16*>(w)[d]);
                                const float wb = p.norm_w_f32 ? static_cast<const float*>(w)[64 + d]
                                                              : __bfloat162float(static_cast<const __nv_bfloat16*>(w)[64 + d]);
                                a = a * inv * wa;
                                b = b * inv * wb;
                            }
                            if (rotate) {
                                const float2 cs = p.cos_sin[(size_t)(ar < p.a_rows ? ar : 0) * 64 + d];
                                const float ra = a * cs.x - b * cs.y, rb2 = a * cs.y + b * cs.x;
                                a = ra; b = rb2;
                            }
                            lo[i] = a; hi[i] = b;
                        }
                        if (dst != nullptr) {
                            store16(dst + c * 16, lo);
                            store16(dst + 64 + c * 16, hi);
                        }
                    }
                }
            } else if (EPI == 1) {
#pragma unroll 1
                for (int c = 0; c < BN / 16; c += 2) {
                    float g[16], u[16];
                    tmem_ld16(lane_addr + c * 16, g);
                    tmem_ld16(lane_addr + (c + 1) * 16, u);
                    const int f0 = b0 + c * 16;
                    if (ar < p.a_rows && f0 + 32 <= p.b_rows) {
                        if (add_bias) {
#pragma unroll
                            for (int i = 0; i < 16; ++i) { g[i] += p.bias[f0 + i]; u[i] += p.bias[f0 + 16 + i]; }
                        }
#pragma unroll
                        for (int i = 0; i < 16; ++i) g[i] = g[i] / (1.f + expf(-g[i])) * u[i];
                        OT* dst = row + (f0 >> 1);
                        if (vec_ok) store16(dst, g);
                        else {
#pragma unroll
                            for (int i = 0; i < 16; ++i) dst[i] = rb::from_f32<OT>(g[i]);
                        }
                    }
                }
            } else if (EPI == 3) {
                // out is the residual stream: out += product.  Every element belongs to one tile and one
                // thread, so nothing else touches it meanwhile; the old values of two column groups are
                // requested before the accumulator is read, so their latency overlaps it.
                if constexpr (std::is_same<OT, float>::value) {
                    rb::pdl_wait();   // these threads read what earlier kernels wrote (the residual): returns at once by now
#pragma unroll 1
                    for (int c = 0; c < BN / 16; c += 2) {
                        const int f0 = b0 + c * 16;
                        const bool whole = vec_ok && f0 + 32 <= p.b_rows && ar < p.a_rows;
                        float r[32];
                        if (whole) {
                            load16(row + f0, r);
                            load16(row + f0 + 16, r + 16);
                        }
                        float v[32];
                        tmem_ld16(lane_addr + c * 16, v);
                        tmem_ld16(lane_addr + (c + 1) * 16, v + 16);
                        if (ar < p.a_rows) {
                            if (add_bias) {
#pragma unroll
                                for (int i = 0; i < 32; ++i) v[i] += (f0 + i < p.b_rows) ? p.bias[f0 + i] : 0.f;
                            }
                            if (whole) {
#pragma unroll
                                for (int i = 0; i < 32; ++i) v[i] += r[i];
                                store16(row + f0, v);
                                store16(row + f0 + 16, v + 16);
                            } else {
#pragma unroll
                                for (int i = 0; i < 32; ++i)
                                    if (f0 + i < p.b_rows) row[f0 + i] += v[i];
                            }
                        }
                    }
                }
} else {
#pragma unroll 1
                for (int c = 0; c < BN / 16; ++c) {
                    float v[16];
                    tmem_ld16(lane_addr + c * 16, v);
                    const int f0 = b0 + c * 16;
                    if (ar < p.a_rows) {
                        if (add_bias) {
#pragma unroll
                            for (int i = 0; i < 16; ++i) v[i] += (f0 + i < p.b_rows) ? p.bias[f0 + i] : 0.f;
                        }
                        if (vec_ok && f0 + 16 <= p.b_rows) {
                            store16(row + f0, v);
                        } else {
#pragma unroll
                            for (int i = 0; i < 16; ++i)
                                if (f0 + i < p.b_rows) row[f0 + i] = rb::from_f32<OT>(v[i]);
                        }
                    }
                }
            }
            // hand the accumulator back to the leader's MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (rank == 0) mbar_arrive(&acc_empty[acc]);
                else mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[acc]), 0));
            }
        }
    }
    // neither CTA may leave while the other can still read its shared memory or signal its barriers
    tc_fence_before();
    __syncthreads();
    cluster_arrive();
    cluster_wait();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

}  // namespace

// ---- host side -------------------------------------------------------------------------------------

namespace {

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

struct MapKey {
    const void* ptr;
    long long rows, K, ld;
    int box_rows;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && K == o.K && ld == o.ld && box_rows == o.box_rows;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = (size_t)k.ptr;
        h = h * 1000003u ^ (size_t)k.rows;
        h = h * 1000003u ^ (size_t)k.K;
        h = h * 1000003u ^ (size_t)k.ld;
        return h * 1000003u ^ (size_t)k.box_rows;
    }
};

// A [rows, K] bf16 matrix with row stride `ld` elements, read in boxes of box_rows x 64 with the
// 128-byte swizzle.  Rows and columns outside the matrix read as zero.  Maps are cached: a
// weight's map is built once.
int tensor_map(const void* ptr, long long rows, long long K, long long ld, int box_rows, CUtensorMap* out) {
    static std::mutex mu;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    MapKey key{ptr, rows, K, ld, box_rows};
    {
        std::lock_guard<std::mutex> g(mu);
        auto it = cache.find(key);
        if (it != cache.end()) { *out = it->second; return RB_OK; }
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return RB_ERR_NO_DRIVER_FN;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return RB_ERR_BAD_SIZE;
    std::lock_guard<std::mutex> g(mu);
    if (cache.size() > 65536) cache.clear();
    cache[key] = *out;
    return RB_OK;
}

template <int BN, bool SWAP, typename OT, bool GATED, int CS = 0>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, void* out, Params p, int splits, cudaStream_t s) {
    // Few tokens (SWAP): the kernel is bound by memory latency, and several small blocks per
    // multiprocessor with a shallow ring hide each other's start and end better than one block
    // with a deep ring (measured: 3 stages beat 5 and 10 on every decode shape).
    if (p.stages <= 0) p.stages = SWAP ? 3 : Cfg<BN>::STAGES;
    using C = Cfg<BN>;
    auto k = gemm_tcgen05_kernel<BN, SWAP, OT, GATED, CS>;
    constexpr int handover_bytes = CS != 0 ? BN * 128 * 4 : 0;
    if (p.stages < 2 || p.stages > C::STAGES) return RB_ERR_BAD_SIZE;
    const int smem_bytes = p.stages * C::STAGE + 1024 + 256 + handover_bytes;
    // The kernel's shared-memory allowance is raised to what a launch needs, no further: how many
    // clusters the device holds at once is worked out from the allowance, not from the launch.
    static int allowance = 0;
    if (smem_bytes > allowance) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        if (e != cudaSuccess) return (int)e;
        if (CS > 8) {   // clusters of more than 8 blocks are not portable
            e = cudaFuncSetAttribute(k, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
            if (e != cudaSuccess) return (int)e;
        }
        allowance = smem_bytes;
    }
    dim3 grid((p.a_rows + BM - 1) / BM, (p.b_rows + BN - 1) / BN, splits);
    if (grid.y > 65535 || grid.z > 65535) return RB_ERR_BAD_SIZE;
    if constexpr (CS != 0) {
        if (splits != CS) return RB_ERR_BAD_SIZE;
        cudaError_t e = rb::launch_clustered(k, grid, dim3(192), dim3(1, 1, CS), smem_bytes, s, ma, mb, (OT*)out, p);
        return e == cudaSuccess ? RB_OK : (int)e;
    } else {
        RB_LAUNCH((k), dim3(grid), dim3(192), smem_bytes, s, ma, mb, (OT*)out, p);
        RB_LAUNCH_CHECK();
        return RB_OK;
    }
}

template <int BN, typename OT, bool GATED>
int launch_persistent(const CUtensorMap& ma, const CUtensorMap& mb, void* out, Params p, cudaStream_t s) {
    using C = Cfg<BN>;
    auto k = gemm_tcgen05_persistent_kernel<BN, OT, GATED>;
    static bool attr_done = false;
    static int sms = 0;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
        if (e != cudaSuccess) return (int)e;
        int dev = 0;
        if ((e = cudaGetDevice(&dev)) != cudaSuccess) return (int)e;
        if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
        attr_done = true;
    }
    if (p.stages <= 0) p.stages = C::STAGES;
    if (p.stages < 2 || p.stages > C::STAGES) return RB_ERR_BAD_SIZE;
    const int smem_bytes = p.stages * C::STAGE + 1024 + 256;
    const long long tiles = (long long)((p.a_rows + BM - 1) / BM) * ((p.b_rows + BN - 1) / BN);
    const int grid = (int)(tiles < sms ? tiles : sms);
    RB_LAUNCH((k), dim3(grid), dim3(192), smem_bytes, s, ma, mb, (OT*)out, p);
    return RB_OK;
}

bool pair_enabled() {
    static const bool on = [] {
        const char* v = std::getenv("RB_GEMM_PAIR");
        return !(v && v[0] == '0');
    }();
    return on;
}

template <typename OT, int EPI>
int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, void* out, Params p, cudaStream_t s) {
    auto k = gemm_tcgen05_pair_kernel<OT, EPI>;
    static bool attr_done = false;
    static int sms = 0;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM);
        if (e != cudaSuccess) return (int)e;
        int dev = 0;
        if ((e = cudaGetDevice(&dev)) != cudaSuccess) return (int)e;
        if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
        attr_done = true;
    }
    const long long tiles = (long long)((p.a_rows + 2 * BM - 1) / (2 * BM)) * ((p.b_rows + PAIR_BN - 1) / PAIR_BN);
    const int pairs = (int)(tiles < sms / 2 ? tiles : sms / 2);
    RB_LAUNCH((k), dim3(2 * pairs), dim3(192), PAIR_SMEM, s, ma, mb, (OT*)out, p);
    return RB_OK;
}

template <bool SWAP, typename OT, bool GATED>
int dispatch_bn(int bn, const CUtensorMap& ma, const CUtensorMap& mb, void* out, const Params& p, int splits,
                cudaStream_t s) {
    switch (bn) {
        case 16: return launch<16, SWAP, OT, GATED>(ma, mb, out, p, splits, s);
        case 32: return launch<32, SWAP, OT, GATED>(ma, mb, out, p, splits, s);
        case 64: return launch<64, SWAP, OT, GATED>(ma, mb, out, p, splits, s);
        case 128: return launch<128, SWAP, OT, GATED>(ma, mb, out, p, splits, s);
        case 256: return launch<256, SWAP, OT, GATED>(ma, mb, out, p, splits, s);
    }
    return RB_ERR_BAD_SIZE;
}

}  // namespace

// out[M, N] (+ splits) = x[M, K] . w[N, K]^T.  x, w bfloat16; out bfloat16 or float32.
// splits > 1: float32 partial results at out + z * split_stride, bias in split 0.
// gated: the weight's rows alternate in blocks of 16 between a gate and an up projection; the output
// is [M, N / 2] = silu(gate) * up (bfloat16, no split).
// Refuses (RB_ERR_BAD_ALIGN) what TMA cannot address: K or ldx not a multiple of 8 elements,
// or a base pointer off a 16-byte boundary; the caller then uses the plain kernel.
struct RopeOut {
    void* q_out; long long q_ld;
    void* k_cache; void* v_cache;
    const int* positions; const int* slot_of_token; const int* block_table; int max_pages;
    const void* q_norm_w; const void* k_norm_w; int norm_w_f32; float norm_eps;
    const float* cos_sin;
    int nq, nkv;
};

struct RowScale {
    const float* sumsq; int groups; long long ld; float eps; int width;
};

struct ResidualOut {
    float* resid; long long resid_ld;
    const void* next_w; int next_w_f32;
    void* xhat; long long xhat_ld;
    float* sumsq; long long sumsq_ld;
};

// The limit of every wait in the kernels of this file, and the tests' switch (see Params); both are
// read when a launch is prepared.
static long long g_wait_cycles = RB_WAIT_CYCLES;
static int g_withhold = 0;

// cycles <= 0 restores the default (about two seconds).  withhold_first_stage != 0 makes the next
// few-token products (at most 128 rows, one split, plain epilogue) skip the copies of their first K
// block, so that the warp that waits for them runs into the limit: for tests of the give-up path,
// with a limit of microseconds.  It computes nothing useful while set.
extern "C" void rb_gemm_tcgen05_set_wait(long long cycles, int withhold_first_stage) {
    g_wait_cycles = cycles > 0 ? cycles : RB_WAIT_CYCLES;
    g_withhold = withhold_first_stage ? 1 : 0;
}

static int gemm_entry(const void* x, const void* w, const float* bias, void* out, int out_dtype, int M,
                      int N, int K, long long ldx, long long ldo, int splits, long long split_stride,
                      int stages, int gated, int* status, void* stream, int cluster_split,
                      const ResidualOut* ro = nullptr, const RowScale* rsc = nullptr, const RopeOut* rope = nullptr,
                      bool accumulate = false) {
    if (M <= 0 || N <= 0) return RB_OK;
    if (K <= 0 || splits < 1) return RB_ERR_BAD_SIZE;
    if (K % 8 || ldx % 8 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return RB_ERR_BAD_ALIGN;
    if (splits > 1 && out_dtype != RB_F32) return RB_ERR_BAD_DTYPE;
    if (gated && (splits != 1 || out_dtype != RB_BF16 || N % 32)) return RB_ERR_BAD_SIZE;
    const int kb_total = (K + BK - 1) / BK;
    if (splits > kb_total) return RB_ERR_BAD_SIZE;  // a split would be empty and its partial result unwritten
    cudaStream_t s = (cudaStream_t)stream;
    const bool swap = M <= 128;
    int bn;
    if (swap) bn = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
    else bn = N >= 256 ? 256 : (N > 64 ? 128 : (N > 32 ? 64 : 32));
    Params p;
    p.K = K;
    p.splits = splits;
    p.ldo = ldo;
    p.split_stride = split_stride;
    p.bias = bias;
    p.status = status;
    p.stages = stages;   // 0: the default of the mode
    p.wait_cycles = g_wait_cycles;
    p.withhold = g_withhold;
    CUtensorMap ma, mb;
    int rc;
    if (swap) {
        p.a_rows = N; p.b_rows = M;
        if ((rc = tensor_map(w, N, K, K, BM, &ma)) != RB_OK) return rc;
        if ((rc = tensor_map(x, M, K, ldx, bn, &mb)) != RB_OK) return rc;
    } else {
        p.a_rows = M; p.b_rows = N;
        if ((rc = tensor_map(x, M, K, ldx, BM, &ma)) != RB_OK) return rc;
        if ((rc = tensor_map(w, N, K, K, bn, &mb)) != RB_OK) return rc;
    }
    p.row_sumsq = nullptr; p.row_groups = 0; p.row_sumsq_ld = 0; p.row_eps = 0.f; p.row_inv_width = 0.f;
    if (rsc != nullptr && rsc->sumsq != nullptr) {
        if (cluster_split != 2 || rsc->groups < 1 || rsc->width < 1) return RB_ERR_BAD_SIZE;
        p.row_sumsq = rsc->sumsq; p.row_groups = rsc->groups; p.row_sumsq_ld = rsc->ld;
        p.row_eps = rsc->eps; p.row_inv_width = 1.f / (float)rsc->width;
    }
    p.resid = nullptr; p.next_w = nullptr; p.xhat = nullptr; p.sumsq = nullptr;
    p.resid_ld = p.xhat_ld = p.sumsq_ld = 0; p.next_w_f32 = 0;
    if (ro != nullptr) {
        if (!swap || bn > 64 || kb_total < cluster_split || ro->resid == nullptr) return RB_ERR_BAD_SIZE;
        if (ro->xhat != nullptr && ro->next_w == nullptr) return RB_ERR_BAD_SIZE;
        p.resid = ro->resid; p.resid_ld = ro->resid_ld;
        p.next_w = ro->next_w; p.next_w_f32 = ro->next_w_f32;
        p.xhat = static_cast<__nv_bfloat16*>(ro->xhat); p.xhat_ld = ro->xhat_ld;
        p.sumsq = ro->sumsq; p.sumsq_ld = ro->sumsq_ld;
        p.splits = cluster_split;
#define RB_RS(BN_)                                                                              \
        switch (cluster_split) {                                                                \
            case 4: return launch<BN_, true, float, false, 4>(ma, mb, nullptr, p, 4, s);        \
            case 8: return launch<BN_, true, float, false, 8>(ma, mb, nullptr, p, 8, s);        \
            case 16: return launch<BN_, true, float, false, 16>(ma, mb, nullptr, p, 16, s);     \
        }                                                                                       \
        return RB_ERR_BAD_SIZE;
        if (bn == 16) { RB_RS(16) }
        if (bn == 32) { RB_RS(32) }
        RB_RS(64)
#undef RB_RS
    }
    if (cluster_split != 0) {
        if (cluster_split != 2 || !swap || bn > 32 || out_dtype != RB_BF16 || N % 32 || kb_total < 2) return RB_ERR_BAD_SIZE;
        p.splits = 2;
        return bn == 16 ? launch<16, true, __nv_bfloat16, false, 2>(ma, mb, out, p, 2, s)
                        : launch<32, true, __nv_bfloat16, false, 2>(ma, mb, out, p, 2, s);
    }
    p.q_out = nullptr; p.k_cache = p.v_cache = nullptr; p.positions = p.slot_of_token = p.block_table = nullptr;
    p.q_norm_w = p.k_norm_w = nullptr; p.cos_sin = nullptr;
    p.q_ld = 0; p.max_pages = 0; p.norm_w_f32 = 0; p.norm_eps = 0.f; p.nq = p.nkv = 0;
    if (rope != nullptr) {
        // a prompt's q | k | v projection: only the kernel of CTA pairs has this epilogue
        if (swap || splits != 1 || bn != 256 || M <= 256 || !pair_enabled() || N % 128 || rope->nq < 1 || rope->nkv < 0 ||
            (N != rope->nq * 128 && N != (rope->nq + 2 * rope->nkv) * 128))
            return RB_ERR_BAD_SIZE;
        if (((uintptr_t)rope->q_out & 15) || (rope->q_ld % 8) || ((uintptr_t)rope->k_cache & 15) || ((uintptr_t)rope->v_cache & 15) ||
            ((uintptr_t)rope->cos_sin & 7))
            return RB_ERR_BAD_ALIGN;
        p.q_out = static_cast<__nv_bfloat16*>(rope->q_out); p.q_ld = rope->q_ld;
        p.k_cache = static_cast<__nv_bfloat16*>(rope->k_cache); p.v_cache = static_cast<__nv_bfloat16*>(rope->v_cache);
        p.positions = rope->positions; p.slot_of_token = rope->slot_of_token; p.block_table = rope->block_table;
        p.max_pages = rope->max_pages;
        p.q_norm_w = rope->q_norm_w; p.k_norm_w = rope->k_norm_w; p.norm_w_f32 = rope->norm_w_f32; p.norm_eps = rope->norm_eps;
        p.cos_sin = reinterpret_cast<const float2*>(rope->cos_sin);
        p.nq = rope->nq; p.nkv = rope->nkv;
        CUtensorMap mb_half;
        if ((rc = tensor_map(w, N, K, K, BM, &mb_half)) != RB_OK) return rc;
        return launch_pair<__nv_bfloat16, 2>(ma, mb_half, nullptr, p, s);
    }
    if (accumulate && (swap || splits != 1 || bn != 256 || M <= 256 || !pair_enabled() || out_dtype != RB_F32 || gated))
        return RB_ERR_BAD_SIZE;            // only the kernel of CTA pairs adds into its output
    if (!swap && splits == 1 && bn == 256 && M > 256 && pair_enabled()) {
        // many tokens and a wide weight: pairs of CTAs; the weight is read in boxes of 128 rows (a half tile)
        CUtensorMap mb_half;
        if ((rc = tensor_map(w, N, K, K, BM, &mb_half)) != RB_OK) return rc;
        if (accumulate) return launch_pair<float, 3>(ma, mb_half, out, p, s);
        if (out_dtype == RB_BF16)
            return gated ? launch_pair<__nv_bfloat16, 1>(ma, mb_half, out, p, s)
                         : launch_pair<__nv_bfloat16, 0>(ma, mb_half, out, p, s);
        if (out_dtype == RB_F32) return launch_pair<float, 0>(ma, mb_half, out, p, s);
    }
    if (!swap && splits == 1 && (bn == 256 || bn == 128)) {
        // many tokens: the persistent kernel with two accumulators (2 x 256 columns fill tensor memory)
        if (out_dtype == RB_BF16) {
            if (bn == 256) return gated ? launch_persistent<256, __nv_bfloat16, true>(ma, mb, out, p, s)
                                        : launch_persistent<256, __nv_bfloat16, false>(ma, mb, out, p, s);
            return gated ? launch_persistent<128, __nv_bfloat16, true>(ma, mb, out, p, s)
                         : launch_persistent<128, __nv_bfloat16, false>(ma, mb, out, p, s);
        }
        if (out_dtype == RB_F32)
            return bn == 256 ? launch_persistent<256, float, false>(ma, mb, out, p, s)
                             : launch_persistent<128, float, false>(ma, mb, out, p, s);
    }
    if (out_dtype == RB_BF16)
    {
        if (gated)
            return swap ? dispatch_bn<true, __nv_bfloat16, true>(bn, ma, mb, out, p, splits, s)
                        : dispatch_bn<false, __nv_bfloat16, true>(bn, ma, mb, out, p, splits, s);
        return swap ? dispatch_bn<true, __nv_bfloat16, false>(bn, ma, mb, out, p, splits, s)
                    : dispatch_bn<false, __nv_bfloat16, false>(bn, ma, mb, out, p, splits, s);
    }
    if (out_dtype == RB_F32)
        return swap ? dispatch_bn<true, float, false>(bn, ma, mb, out, p, splits, s)
                    : dispatch_bn<false, float, false>(bn, ma, mb, out, p, splits, s);
    return RB_ERR_BAD_DTYPE;
}

extern "C" int rb_gemm_tcgen05(const void* x, const void* w, const float* bias, void* out, int out_dtype, int M,
                               int N, int K, long long ldx, long long ldo, int splits, long long split_stride,
                               int stages, int gated, int* status, void* stream) {
    return gemm_entry(x, w, bias, out, out_dtype, M, N, K, ldx, ldo, splits, split_stride, stages, gated, status,
                      stream, 0);
}

// resid[M, N] += x[M, K] . w[N, K]^T (+ bias) for more than 256 rows and N >= 256: the product is added
// into the float32 residual stream (row stride ld_resid) in the epilogue of the kernel of CTA pairs, so
// no delta goes through memory.  RB_ERR_BAD_SIZE for other sizes (the caller writes a delta instead),
// RB_ERR_BAD_ALIGN as rb_gemm_tcgen05.
extern "C" int rb_gemm_tcgen05_add(const void* x, const void* w, const float* bias, float* resid, int M, int N, int K,
                                   long long ldx, long long ld_resid, int stages, int* status, void* stream) {
    return gemm_entry(x, w, bias, resid, RB_F32, M, N, K, ldx, ld_resid, 1, 0, stages, 0, status, stream, 0, nullptr,
                      nullptr, nullptr, true);
}

// h[M, N / 2] = silu(gate) * up (bfloat16, row stride ldh) for at most 32 rows and a gate/up weight
// whose rows alternate in blocks of 16, with the sum over K done in two halves by the two blocks of a
// thread-block cluster (see the kernel).  With row_sumsq (shares [row_groups][>= M] of the sums of squares
// of the rows that x was made from, row_sumsq_ld apart) x is taken as not yet divided by its rows' RMS
// over K values: the product is scaled by rsqrt(sum / K + row_eps) before the bias.
// RB_ERR_BAD_SIZE for more rows, N not a multiple of 32, or K of a single 64-wide block;
// RB_ERR_BAD_ALIGN as rb_gemm_tcgen05.
extern "C" int rb_gemm_tcgen05_gated_pair(const void* x, const void* w, const float* bias, void* h, int M, int N,
                                          int K, long long ldx, long long ldh, const float* row_sumsq,
                                          int row_groups, long long row_sumsq_ld, float row_eps, int stages,
                                          int* status, void* stream) {
    RowScale rsc{row_sumsq, row_groups, row_sumsq_ld, row_eps, K};
    return gemm_entry(x, w, bias, h, RB_BF16, M, N, K, ldx, ldh, 1, 0, stages, 0, status, stream, 2, nullptr, &rsc);
}

// resid[M, N] += x[M, K] . w[N, K]^T (+ bias) for at most 64 rows, the sum over K in `splits` (4, 8
// or 16) parts by the blocks of a thread-block cluster (see the kernel); resid is float32 with row
// stride ld_resid.  For the norm that follows, optionally: xhat[M, N] = bfloat16(resid * next_w)
// (next_w [N], float32 if next_w_f32 else bfloat16) and sumsq[(N / 128) * splits groups][M], each
// group's share of the new rows' sums of squares (group g at sumsq + g * ld_sumsq).
// RB_ERR_BAD_SIZE for more rows or other split counts; RB_ERR_BAD_ALIGN as rb_gemm_tcgen05.
extern "C" int rb_gemm_tcgen05_residual(const void* x, const void* w, const float* bias, int M, int N, int K,
                                        long long ldx, int splits, float* resid, long long ld_resid,
                                        const void* next_w, int next_w_f32, void* xhat, long long ld_xhat,
                                        float* sumsq, long long ld_sumsq, int stages, int* status, void* stream) {
    if (M > 64 || (splits != 4 && splits != 8 && splits != 16)) return RB_ERR_BAD_SIZE;
    ResidualOut ro{resid, ld_resid, next_w, next_w_f32, xhat, ld_xhat, sumsq, ld_sumsq};
    return gemm_entry(x, w, bias, nullptr, RB_F32, M, N, K, ldx, 0, 1, 0, stages, 0, status, stream, splits, &ro);
}

// A prompt's q | k | v projection with heads of 128 (more than 256 rows): x[M, K] . w[N, K]^T (+ bias),
// N = (nq + 2 nkv) * 128, or nq * 128 for a layer that reads another layer's cache.  In the
// product's epilogue every head of every token is normalised (q_norm_w / k_norm_w [128], float32 if
// norm_w_f32 else bfloat16, or null: no norm; values are never normalised) and rotated (cos_sin
// [M][64] pairs, or null), queries go to q_out [M][nq * 128] (row stride q_ld), keys and values into
// their pages (k_cache, v_cache [pages][nkv][64][128]; the page of token t is
// block_table[slot_of_token[t]][positions[t] / 64]; tokens with a negative slot are skipped).
// RB_ERR_BAD_SIZE when the sizes do not fit this kernel (the caller runs the product and the
// rotation kernel one after the other), RB_ERR_BAD_ALIGN as rb_gemm_tcgen05.
extern "C" int rb_gemm_tcgen05_qkv_rope(const void* x, const void* w, const float* bias, int M, int N, int K,
                                        long long ldx, void* q_out, long long q_ld, void* k_cache, void* v_cache,
                                        const int* positions, const int* slot_of_token, const int* block_table,
                                        int max_pages, const void* q_norm_w, const void* k_norm_w, int norm_w_f32,
                                        float norm_eps, const float* cos_sin, int nq, int nkv, int stages,
                                        int* status, void* stream) {
    RopeOut rope{q_out, q_ld, k_cache, v_cache, positions, slot_of_token, block_table, max_pages,
                 q_norm_w, k_norm_w, norm_w_f32, norm_eps, cos_sin, nq, nkv};
    return gemm_entry(x, w, bias, nullptr, RB_BF16, M, N, K, ldx, 0, 1, 0, stages, 0, status, stream, 0, nullptr,
                      nullptr, &rope);
}
