// Sampling on the GPU: one block per sequence of the batch.
//
// rb_argmax: the index of the largest logit, the first one on ties, which is what the
// reference's host sampler returns at temperature <= 0 (rocml/src/sample.rs:172-182).
#include "common.cuh"
#include "api.h"

using namespace rb;

namespace {
struct Best {
    float v;
    int i;
};
__device__ __forceinline__ Best better(Best a, Best b) {
    // larger value wins; on equal values the smaller index wins
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}
__device__ __forceinline__ Best warp_best(Best x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best y;
        y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
        y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
        x = better(x, y);
    }
    return x;
}

__global__ void argmax_kernel(const float* __restrict__ logits, long long row_stride, int V,
                              int* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    __shared__ float sv[32];
    __shared__ int si[32];
    const float* row = logits + (size_t)blockIdx.x * row_stride;
    Best b{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = row[i];
        if (v > b.v) { b.v = v; b.i = i; }  // ascending i per thread: the first maximum stays
    }
    b = warp_best(b);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sv[warp] = b.v; si[warp] = b.i; }
    __syncthreads();
    if (warp == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        Best c{lane < nw ? sv[lane] : -INFINITY, lane < nw ? si[lane] : 0x7fffffff};
        c = warp_best(c);
        if (lane == 0) out[blockIdx.x] = c.i == 0x7fffffff ? 0 : c.i;
    }
}

// Two stages for wide rows: blocks of stage 1 each take a slice of the row, stage 2 (one warp per
// row) picks among their results.  Slices are in index order and ties keep the smaller index, so
// the result is the first maximum, as in the single-block kernel.
__global__ void argmax_partial_kernel(const float* __restrict__ logits, long long row_stride, int V, int per,
                                      float* __restrict__ pv, int* __restrict__ pi) {
    pdl_trigger();
    pdl_wait();
    __shared__ float sv[32];
    __shared__ int si[32];
    const float* row = logits + (size_t)blockIdx.y * row_stride;
    const int lo = blockIdx.x * per, hi = min(V, lo + per);
    Best b{-INFINITY, 0x7fffffff};
    // eight loads a thread in flight, compared in index order: taken one by one each would wait for the one before
    constexpr int UNROLL = 8;
    for (int i0 = lo + threadIdx.x; i0 < hi; i0 += blockDim.x * UNROLL) {
        float v[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int i = i0 + u * blockDim.x;
            v[u] = i < hi ? row[i] : -INFINITY;
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u)
            if (v[u] > b.v) { b.v = v[u]; b.i = i0 + u * blockDim.x; }
    }
    b = warp_best(b);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sv[warp] = b.v; si[warp] = b.i; }
    __syncthreads();
    if (warp == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        Best c{lane < nw ? sv[lane] : -INFINITY, lane < nw ? si[lane] : 0x7fffffff};
        c = warp_best(c);
        if (lane == 0) { pv[blockIdx.y * gridDim.x + blockIdx.x] = c.v; pi[blockIdx.y * gridDim.x + blockIdx.x] = c.i; }
    }
}
__global__ void argmax_final_kernel(const float* __restrict__ pv, const int* __restrict__ pi, int n,
                                    int* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x;
    Best b{-INFINITY, 0x7fffffff};
    for (int i = lane; i < n; i += 32) {
        Best c{pv[blockIdx.x * n + i], pi[blockIdx.x * n + i]};
        b = better(b, c);
    }
    b = warp_best(b);
    if (lane == 0) out[blockIdx.x] = b.i == 0x7fffffff ? 0 : b.i;
}
}  // namespace

// scratch_v / scratch_i: [rows, slices] work space for rows wider than 8192; slices > 1 selects the
// two-stage route.
extern "C" int rb_argmax(const float* logits, long long row_stride, int rows, int V, int* out, float* scratch_v,
                         int* scratch_i, int slices, void* stream) {
    if (rows <= 0) return RB_OK;
    if (V <= 0) return RB_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (slices > 1 && scratch_v && scratch_i) {
        if (rows > 65535) return RB_ERR_BAD_SIZE;
        const int per = (V + slices - 1) / slices;
        RB_LAUNCH((argmax_partial_kernel), dim3(dim3(slices, rows)), dim3(256), 0, s, logits, row_stride, V, per, scratch_v, scratch_i);
        RB_LAUNCH_CHECK();
        RB_LAUNCH((argmax_final_kernel), dim3(rows), dim3(32), 0, s, scratch_v, scratch_i, slices, out);
        RB_LAUNCH_CHECK();
        return RB_OK;
    }
    RB_LAUNCH((argmax_kernel), dim3(rows), dim3(1024), 0, s, logits, row_stride, V, out);
    RB_LAUNCH_CHECK();
    return RB_OK;
}

// ---- temperature / top-k / top-p / repeat penalty / draw -------------------------------------------
//
// rb_sample follows the reference's host sampler step by step (rocml/src/sample.rs:90-166):
// repeat penalty over the last `window` history ids, once per occurrence (:188-202) ->
// temperature <= 0: argmax (:172-182) -> logits * (1 / temperature) (:102-105) -> keep the
// top_k largest (:110-116) -> softmax over the survivors with the maximum subtracted (:118-131)
// -> top_p: survivors in descending order, shortest prefix whose cumulative probability reaches
// top_p, at least one (:138-153) -> threshold = u * (sum of the kept probabilities); walk the
// kept candidates (descending order if top_p was applied, else index order) until the running
// sum reaches it (:155-165).  The uniform number u comes from the host's xorshift64* stream,
// so a seed gives the same draws as the reference's generator.
//
// Two routes, both deterministic:
//  * top_k given and at most 1024 candidates survive it: the candidates are gathered in shared
//    memory, sorted (by value, or by index when there is no top_p) and walked by one thread in
//    float32, exactly the reference's arithmetic up to the order of the softmax sum.
//  * otherwise thresholds are found by radix selection over the whole row, with probabilities
//    as 40-bit fixed-point integers so that sums do not depend on the order of the atomics.
// Logits that tie exactly with the top_k threshold are all kept (the reference keeps an
// arbitrary subset of them); ties at the top_p threshold and at the drawn value are taken one
// by one in index order.
namespace {

struct SampleRow {
    float temperature;
    int top_k;        // 0: off
    float top_p;      // < 0: off
    float u;          // uniform in [0, 1)
    float penalty;    // <= 0: off
    int hist_begin;   // into the history buffer
    int hist_len;
    int pad;
};

constexpr int ST = 1024;          // threads per row
constexpr int MAX_CAND = 1024;    // candidates the shared-memory route holds
constexpr float FIX = 1099511627776.0f;  // 2^40

__device__ __forceinline__ uint32_t key_of(float v) {
    const uint32_t b = __float_as_uint(v);
    return b ^ ((b >> 31) ? 0xffffffffu : 0x80000000u);  // ascending in the float's order
}
__device__ __forceinline__ unsigned long long fixed_of(float p) {
    return (unsigned long long)(p * FIX);
}

// Every element of a row is handed to f(index, value) once, by some thread, in no particular order.
// One block reads the row, and what bounds it is how many bytes it keeps in flight: four 16-byte
// loads a thread are requested before the first element is worked on (rows that are not 16-byte
// aligned or whose length is no multiple of 4 fall back to single elements).
template <typename F>
__device__ __forceinline__ void for_each_strided(const float* row, int V, int tid, F f) {
    if ((((uintptr_t)row & 15) | (V & 3)) == 0) {
        const float4* r4 = reinterpret_cast<const float4*>(row);
        const int V4 = V >> 2;
        int i = tid;
        for (; i + 3 * ST < V4; i += 4 * ST) {
            const float4 a = r4[i], b = r4[i + ST], c = r4[i + 2 * ST], d = r4[i + 3 * ST];
            f(4 * i, a.x); f(4 * i + 1, a.y); f(4 * i + 2, a.z); f(4 * i + 3, a.w);
            f(4 * (i + ST), b.x); f(4 * (i + ST) + 1, b.y); f(4 * (i + ST) + 2, b.z); f(4 * (i + ST) + 3, b.w);
            f(4 * (i + 2 * ST), c.x); f(4 * (i + 2 * ST) + 1, c.y); f(4 * (i + 2 * ST) + 2, c.z); f(4 * (i + 2 * ST) + 3, c.w);
            f(4 * (i + 3 * ST), d.x); f(4 * (i + 3 * ST) + 1, d.y); f(4 * (i + 3 * ST) + 2, d.z); f(4 * (i + 3 * ST) + 3, d.w);
        }
        for (; i < V4; i += ST) {
            const float4 a = r4[i];
            f(4 * i, a.x); f(4 * i + 1, a.y); f(4 * i + 2, a.z); f(4 * i + 3, a.w);
        }
        return;
    }
    int i = tid;
    for (; i + 3 * ST < V; i += 4 * ST) {
        const float a = row[i], b = row[i + ST], c = row[i + 2 * ST], d = row[i + 3 * ST];
        f(i, a); f(i + ST, b); f(i + 2 * ST, c); f(i + 3 * ST, d);
    }
    for (; i < V; i += ST) f(i, row[i]);
}

// hist[bucket] += w in shared memory with 32-bit atomics only (64-bit ones are slow under the
// contention a histogram sees): the low word takes the low half, and the high word is touched only
// when the weight has a high half or the low word wrapped, which is rare.  Exact whatever the order.
__device__ __forceinline__ void hist_add(unsigned long long* hist, int bucket, unsigned long long w) {
    unsigned int* words = reinterpret_cast<unsigned int*>(hist + bucket);      // little-endian: [0] low, [1] high
    const unsigned int lo = (unsigned int)w, hi = (unsigned int)(w >> 32);
    const unsigned int old = atomicAdd(words, lo);
    const unsigned int carry = old + lo < old ? 1u : 0u;
    if (hi + carry) atomicAdd(words + 1, hi + carry);
}

struct Shared {
    unsigned long long hist[256];
    unsigned long long scan[ST / 32];
    float cand_val[MAX_CAND];
    float cand_p[MAX_CAND];
    int cand_idx[MAX_CAND];
    float red_v[32];
    int red_i[32];
    unsigned long long acc;
    int chosen;
    int count;
    int flag;
};

// ---- a row shared by the blocks of a cluster ------------------------------------------------------
// One block reads a row of 150,000 logits at a small fraction of the device's bandwidth, and a sampler
// makes eight or so passes over it.  So the row is cut into C contiguous parts, one per block of a
// thread-block cluster; every pass runs on the parts side by side, and what a pass finds (a maximum, a
// sum, a histogram) is combined through distributed shared memory so that EVERY block holds the same
// result and takes the same decisions.  C = 1 is the plain one-block kernel.
template <int C>
struct Team {
    unsigned rank;
    __device__ void barrier() const {
        if (C > 1) {
            asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
            asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        } else {
            __syncthreads();
        }
    }
    template <typename T>
    __device__ T peer(const T* local, unsigned r) const {          // the value `local` has in block r
        if (C == 1) return *local;
        uint32_t remote;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
                     : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(r));
        T v;
        if (sizeof(T) == 8) {
            unsigned long long raw;
            asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(raw) : "r"(remote) : "memory");
            v = *reinterpret_cast<T*>(&raw);
        } else {
            unsigned int raw;
            asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(raw) : "r"(remote) : "memory");
            v = *reinterpret_cast<T*>(&raw);
        }
        return v;
    }
    // every block's *value (written by one of its threads before the call) -> the sum over the blocks, in
    // every block
    template <typename T>
    __device__ T sum(T* value) const {
        barrier();
        T t = 0;
        for (unsigned r = 0; r < (unsigned)C; ++r) t += peer(value, r);
        barrier();                                                  // everyone has read before anyone writes again
        return t;
    }
    // every block's histogram -> their sum, in every block
    __device__ void sum_hist(unsigned long long* hist) const {
        if (C == 1) { __syncthreads(); return; }
        barrier();
        unsigned long long t = 0;
        if (threadIdx.x < 256)
            for (unsigned r = 0; r < (unsigned)C; ++r) t += peer(&hist[threadIdx.x], r);
        barrier();
        if (threadIdx.x < 256) hist[threadIdx.x] = t;
        __syncthreads();
    }
};

// A coarse ranking that every pass computes the same way from the value alone: how far below the row's
// maximum the (scaled) logit lies, in eighths, 255 for everything 32 or more below.  Smaller = larger.
__device__ __forceinline__ int coarse_bin(float s, float max_s) {
    const float d = (max_s - s) * 8.f;
    return d >= 255.f ? 255 : (d > 0.f ? (int)d : 0);
}

// Where the running sum over the 256 bins, started at `above` (< target), reaches `target`: bins taken
// from 255 down (descending) or from 0 up; the last bin in that order is the answer if no earlier one is.
// One thread a bin and a scan over them.  Leaves the bin in sh.chosen and the sum before it in sh.acc,
// for every thread.
__device__ __forceinline__ void find_bin(Shared& sh, unsigned long long above, unsigned long long target,
                                         bool descending) {
    const int j = threadIdx.x, lane = j & 31;
    unsigned long long v = 0, incl = 0;
    if (j < 256) {
        v = sh.hist[descending ? 255 - j : j];
        incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned long long up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
        if (lane == 31) sh.scan[j >> 5] = incl;
    }
    __syncthreads();
    if (j < 256) {
        for (int w = 0; w < (j >> 5); ++w) incl += sh.scan[w];
        const unsigned long long before = above + incl - v;
        if (before < target && (above + incl >= target || j == 255)) {      // true for exactly one bin
            sh.chosen = descending ? 255 - j : j;
            sh.acc = before;
        }
    }
    __syncthreads();
}

// Threshold key T with weight(key > T) < target <= weight(key >= T) over the elements whose
// key is >= min_key; weight is 1 (BY_MASS = false) or the fixed-point probability.
// `part` is this block's part of the row (n elements).  *w_greater: weight(key > T); *w_equal:
// weight(key == T).
template <bool BY_MASS, int C>
__device__ uint32_t radix_select(const Team<C>& team, const float* part, int n, float inv_temp, float max_s,
                                 uint32_t min_key, unsigned long long target, Shared& sh,
                                 unsigned long long* w_greater, unsigned long long* w_equal) {
    // First a histogram over the coarse bins.  The logits of a row share a few exponents, so a
    // radix pass over the keys' top bits piles every atomic onto a handful of counters; the distance
    // below the maximum spreads them over the bins, and the bin that holds the threshold is found with
    // one pass.  That bin's elements are then copied to shared memory, and the radix passes over the
    // key's bytes run on the copy (on the row itself if some block's share of the bin does not fit).
    const int tid = threadIdx.x;
    if (tid < 256) sh.hist[tid] = 0;
    if (tid == 0) sh.count = 0;
    __syncthreads();
    for_each_strided(part, n, tid, [&](int, float v) {
        const float s = v * inv_temp;
        if (key_of(s) >= min_key) hist_add(sh.hist, coarse_bin(s, max_s), BY_MASS ? fixed_of(expf(s - max_s)) : 1ull);
    });
    team.sum_hist(sh.hist);
    find_bin(sh, 0ull, target, false);                      // bin 0 holds the largest values
    const int bin = sh.chosen;
    unsigned long long above = sh.acc;
    for_each_strided(part, n, tid, [&](int, float v) {
        const float s = v * inv_temp;
        if (key_of(s) >= min_key && coarse_bin(s, max_s) == bin) {
            const int pos = atomicAdd(&sh.count, 1);
            if (pos < MAX_CAND) sh.cand_val[pos] = s;
        }
    });
    __syncthreads();
    const int n_list = sh.count;
    if (tid == 0) sh.flag = n_list > MAX_CAND;
    const bool listed = team.sum(&sh.flag) == 0;            // the same answer in every block
    uint32_t prefix = 0, mask = 0;
    unsigned long long equal = 0;
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        if (tid < 256) sh.hist[tid] = 0;
        __syncthreads();
        if (listed) {
            for (int j = tid; j < n_list; j += ST) {
                const float s = sh.cand_val[j];
                const uint32_t key = key_of(s);
                if ((key & mask) == prefix)
                    hist_add(sh.hist, (int)((key >> shift) & 255u), BY_MASS ? fixed_of(expf(s - max_s)) : 1ull);
            }
        } else {
            for_each_strided(part, n, tid, [&](int, float v) {
                const float s = v * inv_temp;
                const uint32_t key = key_of(s);
                if (key >= min_key && (key & mask) == prefix && coarse_bin(s, max_s) == bin)
                    hist_add(sh.hist, (int)((key >> shift) & 255u), BY_MASS ? fixed_of(expf(s - max_s)) : 1ull);
            });
        }
        team.sum_hist(sh.hist);
        find_bin(sh, above, target, true);
        prefix |= (uint32_t)sh.chosen << shift;
        mask |= 255u << shift;
        above = sh.acc;
        equal = sh.hist[sh.chosen];
        __syncthreads();
    }
    *w_greater = above;
    *w_equal = equal;
    return prefix;
}


// Walk the row in index order and write to *out the first index at which the running weight reaches
// thr (>= 1), or `fallback` if it never does.  MODE 0: weight = fixed-point probability of elements with
// key >= key_ref; MODE 1: weight = 1 for elements with key == key_ref.  Every warp sums one contiguous
// stretch of its block's part (its lanes side by side, so the reads coalesce), the stretches' sums are
// scanned over the warps and over the blocks, and the one warp whose stretch holds the crossing walks
// it 256 elements at a time with a scan across its lanes.  The weights are integers, so no sum depends
// on the order it was formed in.  `first` is the row index of the part's first element.
template <int MODE, int C>
__device__ void index_walk(const Team<C>& team, const float* part, int n, int first, float inv_temp, float max_s,
                           uint32_t key_ref, unsigned long long thr, Shared& sh, int fallback, int* out) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int WARPS_ = ST / 32;
    const int per = ((n + WARPS_ - 1) / WARPS_ + 31) & ~31;        // a warp's stretch, a multiple of 32
    const int lo = warp * per, hi = min(n, lo + per);
    auto weight = [&](int i) -> unsigned long long {
        if (i >= hi) return 0ull;
        const float s = part[i] * inv_temp;
        const uint32_t key = key_of(s);
        if (MODE == 0) return key >= key_ref ? fixed_of(expf(s - max_s)) : 0ull;
        return key == key_ref ? 1ull : 0ull;
    };
    unsigned long long mine = 0;
    for (int i = lo + lane; i < hi; i += 32) mine += weight(i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
    __syncthreads();
    if (lane == 0) sh.scan[warp] = mine;
    __syncthreads();
    unsigned long long before = 0, block_total = 0;
    for (int w = 0; w < WARPS_; ++w) {
        if (w < warp) before += sh.scan[w];
        block_total += sh.scan[w];
    }
    if (tid == 0) {
        sh.acc = block_total;
        if (team.rank == 0) *out = fallback;                        // stands unless a warp finds the crossing
    }
    team.barrier();                                                 // the blocks' totals are there; the fallback is written
    for (unsigned r = 0; r < team.rank; ++r) before += team.peer(&sh.acc, r);
    if (before < thr && thr <= before + mine) {                   // this warp's stretch holds the crossing
        // 256 elements at a time, 8 neighbours a lane: the loads of a round are all in flight together
        unsigned long long run = before;
        for (int base = lo; base < hi; base += 256) {
            unsigned long long w[8], sum = 0;
#pragma unroll
            for (int k = 0; k < 8; ++k) { w[k] = weight(base + lane * 8 + k); sum += w[k]; }
            unsigned long long incl = sum;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned long long up = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += up;
            }
            const unsigned long long round = __shfl_sync(0xffffffffu, incl, 31);
            if (run + round >= thr) {
                unsigned long long cum = run + incl - sum;
                if (cum < thr && thr <= cum + sum) {
                    int k = 0;
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        if (cum < thr) { cum += w[q]; k = q; }
                    }
                    *out = first + base + lane * 8 + k;
                }
                break;
            }
            run += round;
        }
    }
    team.barrier();                                                 // nobody leaves while its total may still be read
}

__device__ __forceinline__ float value_of_key(uint32_t key) {
    const uint32_t b = (key & 0x80000000u) ? (key ^ 0x80000000u) : ~key;
    return __uint_as_float(b);
}

__device__ __forceinline__ bool cand_before(float va, int ia, float vb, int ib, bool by_value) {
    if (by_value) return va > vb || (va == vb && ia < ib);
    return ia < ib;
}

template <int C>
__global__ void __launch_bounds__(ST, 2)
sample_kernel(float* __restrict__ logits, long long row_stride, int V, const SampleRow* __restrict__ rows,
              const int* __restrict__ history, int* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    __shared__ Shared sh;
    const int row_id = blockIdx.x / C;
    Team<C> team;
    team.rank = blockIdx.x % C;                               // = the block's rank in its cluster of C
    const SampleRow r = rows[row_id];
    float* row = logits + (size_t)row_id * row_stride;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // this block's part of the row: a multiple of 4 elements, so that 16-byte loads stay aligned
    const int per = (((V + C - 1) / C) + 3) & ~3;
    const int first = min(V, (int)team.rank * per);
    const int n = min(V, first + per) - first;
    const float* part = row + first;
    int* result = out + row_id;

    // repeat penalty, once per occurrence, in history order
    if (r.penalty > 0.f && fabsf(r.penalty - 1.f) >= 1.1920929e-7f) {
        if (tid == 0 && team.rank == 0) {
            for (int j = 0; j < r.hist_len; ++j) {
                const int id = history[r.hist_begin + j];
                if (id >= 0 && id < V) row[id] = row[id] > 0.f ? row[id] / r.penalty : row[id] * r.penalty;
            }
            __threadfence();
        }
        team.barrier();
    }

    // the largest logit, first index on ties
    Best b{-INFINITY, 0x7fffffff};
    for_each_strided(part, n, tid, [&](int i, float v) {
        if (v > b.v) { b.v = v; b.i = first + i; }
    });
    b = warp_best(b);
    if (lane == 0) { sh.red_v[warp] = b.v; sh.red_i[warp] = b.i; }
    __syncthreads();
    if (warp == 0) {
        Best c{sh.red_v[lane], sh.red_i[lane]};
        c = warp_best(c);
        if (lane == 0) { sh.red_v[0] = c.v; sh.red_i[0] = c.i; }
    }
    team.barrier();
    Best top{-INFINITY, 0x7fffffff};
    for (unsigned q = 0; q < (unsigned)C; ++q) top = better(top, Best{team.peer(&sh.red_v[0], q), team.peer(&sh.red_i[0], q)});
    team.barrier();
    const float max_logit = top.v;
    const int arg = top.i == 0x7fffffff ? 0 : top.i;
    if (r.temperature <= 0.f) {
        if (tid == 0 && team.rank == 0) *result = arg;
        return;                                               // every block of the cluster takes this way together
    }
    const float inv_temp = 1.0f / r.temperature;
    const float max_s = max_logit * inv_temp;
    const bool use_p = r.top_p >= 0.f;
    const float top_p = fminf(fmaxf(r.top_p, 0.f), 1.f);

    uint32_t min_key = 0;
    unsigned long long n_keep = (unsigned long long)V;
    if (r.top_k > 0 && r.top_k < V) {
        // how many reach the threshold (ties included) comes out of the selection itself
        unsigned long long greater, equal;
        min_key = radix_select<false>(team, part, n, inv_temp, max_s, 0u, (unsigned long long)r.top_k, sh, &greater, &equal);
        n_keep = greater + equal;
    }

    if (r.top_k > 0 && n_keep <= (unsigned long long)MAX_CAND) {
        // ---- route 1: candidates in shared memory ----------------------------------------------
        if (tid == 0) sh.count = 0;
        sh.cand_val[tid] = -INFINITY;
        sh.cand_idx[tid] = 0x7fffffff;
        __syncthreads();
        for_each_strided(part, n, tid, [&](int i, float v) {
            const float s = v * inv_temp;
            if (key_of(s) >= min_key) {
                const int pos = atomicAdd(&sh.count, 1);
                sh.cand_val[pos] = s;
                sh.cand_idx[pos] = first + i;
            }
        });
        team.barrier();
        if (team.rank == 0) {
            // the other blocks' candidates come over; the order does not matter, the sort below settles it
            int have = sh.count;
            for (unsigned q = 1; q < (unsigned)C; ++q) {
                const int theirs = team.peer(&sh.count, q);
                for (int j = tid; j < theirs; j += ST) {
                    sh.cand_val[have + j] = team.peer(&sh.cand_val[j], q);
                    sh.cand_idx[have + j] = team.peer(&sh.cand_idx[j], q);
                }
                have += theirs;
            }
            __syncthreads();
            const int total = have;
            // bitonic sort, one entry per thread, of the smallest power of two that holds the candidates;
            // empty entries sort last.  Up to 32 entries are one warp's own business.
            int sort_n = 32;
            while (sort_n < total) sort_n <<= 1;
            auto exchange = [&](int size, int stride) {
                const int partner = tid ^ stride;
                if (partner > tid && partner < sort_n) {
                    const bool up = (tid & size) == 0;
                    const float va = sh.cand_val[tid], vb = sh.cand_val[partner];
                    const int ia = sh.cand_idx[tid], ib = sh.cand_idx[partner];
                    const bool a_first = cand_before(va, ia, vb, ib, use_p);
                    if (a_first != up) {
                        sh.cand_val[tid] = vb; sh.cand_val[partner] = va;
                        sh.cand_idx[tid] = ib; sh.cand_idx[partner] = ia;
                    }
                }
            };
            if (sort_n == 32) {
                if (warp == 0) {
                    for (int size = 2; size <= 32; size <<= 1)
                        for (int stride = size >> 1; stride > 0; stride >>= 1) {
                            exchange(size, stride);
                            __syncwarp();
                        }
                }
                __syncthreads();
            } else {
                for (int size = 2; size <= sort_n; size <<= 1)
                    for (int stride = size >> 1; stride > 0; stride >>= 1) {
                        exchange(size, stride);
                        __syncthreads();
                    }
            }
            if (tid == 0) {
                float sum = 0.f;
                for (int j = 0; j < total; ++j) { sh.cand_p[j] = expf(sh.cand_val[j] - max_s); sum += sh.cand_p[j]; }
                if (sum > 0.f) for (int j = 0; j < total; ++j) sh.cand_p[j] /= sum;
                int keep = total;
                float eff = 0.f;
                if (use_p) {
                    float cum = 0.f;
                    for (int j = 0; j < total; ++j) {
                        cum += sh.cand_p[j];
                        if (cum >= top_p) { keep = j + 1; break; }
                    }
                    keep = keep < 1 ? 1 : keep;
                }
                for (int j = 0; j < keep; ++j) eff += sh.cand_p[j];
                const float thr = r.u * fmaxf(eff, 1.17549435e-38f);
                float acc = 0.f;
                int pick = sh.cand_idx[0];
                for (int j = 0; j < keep; ++j) {
                    acc += sh.cand_p[j];
                    if (acc >= thr) { pick = sh.cand_idx[j]; break; }
                }
                *result = pick;
            }
        }
        team.barrier();                                       // the others stay until their candidates have been read
        return;
    }

    // ---- route 2: thresholds by radix selection over the whole row ------------------------------
    // total mass of the kept candidates
    unsigned long long mass = 0;
    for_each_strided(part, n, tid, [&](int, float v) {
        const float s = v * inv_temp;
        if (key_of(s) >= min_key) mass += fixed_of(expf(s - max_s));
    });
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mass += __shfl_xor_sync(0xffffffffu, mass, o);
    __syncthreads();
    if (lane == 0) sh.scan[warp] = mass;
    __syncthreads();
    if (tid == 0) {
        unsigned long long t = 0;
        for (int w = 0; w < ST / 32; ++w) t += sh.scan[w];
        sh.acc = t;
    }
    unsigned long long eff = team.sum(&sh.acc);   // >= 2^40: the maximum itself has probability weight 1
    if (use_p) {
        unsigned long long target = (unsigned long long)((double)top_p * (double)eff);
        target = target < 1 ? 1 : (target > eff ? eff : target);
        unsigned long long greater, equal;
        const uint32_t tp = radix_select<true>(team, part, n, inv_temp, max_s, min_key, target, sh, &greater, &equal);
        min_key = tp > min_key ? tp : min_key;
        // candidates that tie with the threshold enter one by one, in index order, until the
        // cumulative mass reaches the target
        const unsigned long long q = fixed_of(expf(value_of_key(tp) - max_s));
        const unsigned long long ties = q ? (target - greater + q - 1) / q : 1;
        eff = greater + ties * q;
    }
    unsigned long long thr = (unsigned long long)((double)r.u * (double)eff);
    thr = thr < 1 ? 1 : (thr > eff ? eff : thr);
    if (use_p) {
        // walk in descending order: the value at which the mass from the top reaches thr, then the
        // j-th candidate of that value in index order
        unsigned long long greater, equal;
        const uint32_t td = radix_select<true>(team, part, n, inv_temp, max_s, min_key, thr, sh, &greater, &equal);
        const unsigned long long q = fixed_of(expf(value_of_key(td) - max_s));
        const unsigned long long j = q ? (thr - greater + q - 1) / q : 1;
        index_walk<1>(team, part, n, first, inv_temp, max_s, td, j < 1 ? 1 : j, sh, arg, result);
    } else {
        index_walk<0>(team, part, n, first, inv_temp, max_s, min_key, thr, sh, arg, result);
    }
}
}  // namespace

// rows: [n] records of 8 x 4 bytes {temperature, top_k, top_p (<0 off), u, penalty (<=0 off),
// hist_begin, hist_len, 0}; history: int32 ids.  logits are modified in place by the penalty.
extern "C" int rb_sample(float* logits, long long row_stride, int n, int V, const void* rows, const int* history,
                         int* out, void* stream) {
    if (n <= 0) return RB_OK;
    if (V <= 0) return RB_ERR_BAD_SIZE;
    // wide rows: eight blocks a row, as a cluster (see Team)
    constexpr int TEAM = 8;
    if (V >= 16384) {
        cudaError_t e = rb::launch_clustered(sample_kernel<TEAM>, dim3(n * TEAM), dim3(ST), dim3(TEAM, 1, 1), 0,
                                             (cudaStream_t)stream, logits, row_stride, V, (const SampleRow*)rows, history, out);
        return e == cudaSuccess ? RB_OK : (int)e;
    }
    RB_LAUNCH((sample_kernel<1>), dim3(n), dim3(ST), 0, (cudaStream_t)stream, logits, row_stride, V, (const SampleRow*)rows, history, out);
    RB_LAUNCH_CHECK();
    return RB_OK;
}
