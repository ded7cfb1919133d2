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
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = row[i];
        if (v > b.v) { b.v = v; b.i = i; }
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

// Every thread visits the elements tid, tid + ST, ... of a row; four loads are issued before the
// first element is worked on (a pass over a row is bound by the latency of its loads otherwise).
template <typename F>
__device__ __forceinline__ void for_each_strided(const float* row, int V, int tid, F f) {
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
    unsigned long long scan[ST];
    float cand_val[MAX_CAND];
    float cand_p[MAX_CAND];
    int cand_idx[MAX_CAND];
    float red_v[32];
    int red_i[32];
    unsigned long long acc;
    int chosen;
    int count;
    int token;
};

// Threshold key T with weight(key > T) < target <= weight(key >= T) over the elements whose
// key is >= min_key; weight is 1 (BY_MASS = false) or the fixed-point probability.
// A coarse ranking that every pass computes the same way from the value alone: how far below the row's
// maximum the (scaled) logit lies, in eighths, 255 for everything 32 or more below.  Smaller = larger.
__device__ __forceinline__ int coarse_bin(float s, float max_s) {
    const float d = (max_s - s) * 8.f;
    return d >= 255.f ? 255 : (d > 0.f ? (int)d : 0);
}

template <bool BY_MASS>
__device__ uint32_t radix_select(const float* row, int V, float inv_temp, float max_s, uint32_t min_key,
                                 unsigned long long target, Shared& sh, unsigned long long* w_greater) {
    // First a histogram over the coarse bins.  The logits of a row share a few exponents, so a
    // radix pass over the keys' top bits piles every atomic onto a handful of counters; the distance
    // below the maximum spreads them over the bins, and the bin that holds the threshold is found with
    // one pass.  The radix passes that follow only look at that bin's few elements.
    if (threadIdx.x < 256) sh.hist[threadIdx.x] = 0;
    __syncthreads();
    for_each_strided(row, V, threadIdx.x, [&](int, float v) {
        const float s = v * inv_temp;
        if (key_of(s) >= min_key) {
            hist_add(sh.hist, coarse_bin(s, max_s), BY_MASS ? fixed_of(expf(s - max_s)) : 1ull);
        }
    });
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long acc = 0;
        int b = 0;
        for (; b < 255; ++b) {                              // bin 0 holds the largest values
            if (acc + sh.hist[b] >= target) break;
            acc += sh.hist[b];
        }
        sh.chosen = b;
        sh.acc = acc;
    }
    __syncthreads();
    const int bin = sh.chosen;
    uint32_t prefix = 0, mask = 0;
    unsigned long long above = sh.acc;
    __syncthreads();
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        if (threadIdx.x < 256) sh.hist[threadIdx.x] = 0;
        __syncthreads();
        for_each_strided(row, V, threadIdx.x, [&](int, float v) {
            const float s = v * inv_temp;
            const uint32_t key = key_of(s);
            if (key >= min_key && (key & mask) == prefix && coarse_bin(s, max_s) == bin) {
                hist_add(sh.hist, (int)((key >> shift) & 255u), BY_MASS ? fixed_of(expf(s - max_s)) : 1ull);
            }
        });
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned long long acc = above;
            int b = 255;
            for (; b > 0; --b) {
                if (acc + sh.hist[b] >= target) break;
                acc += sh.hist[b];
            }
            sh.chosen = b;
            sh.acc = acc;
        }
        __syncthreads();
        prefix |= (uint32_t)sh.chosen << shift;
        mask |= 255u << shift;
        above = sh.acc;
        __syncthreads();
    }
    *w_greater = above;
    return prefix;
}


// Walk the row in index order and return the first index at which the running weight reaches
// thr (>= 1).  MODE 0: weight = fixed-point probability of elements with key >= key_ref;
// MODE 1: weight = 1 for elements with key == key_ref.  Each thread sums a contiguous range,
// the ranges are scanned, and the thread whose range holds the crossing walks it.
template <int MODE>
__device__ int index_walk(const float* row, int V, float inv_temp, float max_s, uint32_t key_ref,
                          unsigned long long thr, Shared& sh, int fallback) {
    const int tid = threadIdx.x;
    const int per = (V + ST - 1) / ST;
    const int lo = tid * per, hi = min(V, lo + per);
    unsigned long long part = 0;
    for (int i = lo; i < hi; ++i) {
        const float s = row[i] * inv_temp;
        const uint32_t key = key_of(s);
        if (MODE == 0) { if (key >= key_ref) part += fixed_of(expf(s - max_s)); }
        else { if (key == key_ref) part += 1; }
    }
    __syncthreads();
    sh.scan[tid] = part;
    if (tid == 0) sh.token = 0x7fffffff;
    __syncthreads();
    if (tid == 0) {
        unsigned long long run = 0;
        for (int t = 0; t < ST; ++t) { const unsigned long long v = sh.scan[t]; sh.scan[t] = run; run += v; }
    }
    __syncthreads();
    const unsigned long long before = sh.scan[tid];
    if (before < thr && thr <= before + part) {
        unsigned long long run = before;
        for (int i = lo; i < hi; ++i) {
            const float s = row[i] * inv_temp;
            const uint32_t key = key_of(s);
            unsigned long long w = 0;
            if (MODE == 0) { if (key >= key_ref) w = fixed_of(expf(s - max_s)); }
            else { if (key == key_ref) w = 1; }
            run += w;
            if (w && run >= thr) { sh.token = i; break; }
        }
    }
    __syncthreads();
    const int tok = sh.token == 0x7fffffff ? fallback : sh.token;
    __syncthreads();
    return tok;
}

__device__ __forceinline__ float value_of_key(uint32_t key) {
    const uint32_t b = (key & 0x80000000u) ? (key ^ 0x80000000u) : ~key;
    return __uint_as_float(b);
}

__device__ __forceinline__ bool cand_before(float va, int ia, float vb, int ib, bool by_value) {
    if (by_value) return va > vb || (va == vb && ia < ib);
    return ia < ib;
}

__global__ void __launch_bounds__(ST)
sample_kernel(float* __restrict__ logits, long long row_stride, int V, const SampleRow* __restrict__ rows,
              const int* __restrict__ history, int* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    __shared__ Shared sh;
    const SampleRow r = rows[blockIdx.x];
    float* row = logits + (size_t)blockIdx.x * row_stride;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    // repeat penalty, once per occurrence, in history order
    if (r.penalty > 0.f && fabsf(r.penalty - 1.f) >= 1.1920929e-7f && tid == 0) {
        for (int j = 0; j < r.hist_len; ++j) {
            const int id = history[r.hist_begin + j];
            if (id >= 0 && id < V) row[id] = row[id] > 0.f ? row[id] / r.penalty : row[id] * r.penalty;
        }
    }
    __syncthreads();

    // the largest logit, first index on ties
    Best b{-INFINITY, 0x7fffffff};
    for_each_strided(row, V, tid, [&](int i, float v) {
        if (v > b.v) { b.v = v; b.i = i; }
    });
    b = warp_best(b);
    if (lane == 0) { sh.red_v[warp] = b.v; sh.red_i[warp] = b.i; }
    __syncthreads();
    if (warp == 0) {
        Best c{sh.red_v[lane], sh.red_i[lane]};
        c = warp_best(c);
        if (lane == 0) { sh.red_v[0] = c.v; sh.red_i[0] = c.i == 0x7fffffff ? 0 : c.i; }
    }
    __syncthreads();
    const float max_logit = sh.red_v[0];
    const int arg = sh.red_i[0];
    __syncthreads();
    if (r.temperature <= 0.f) {
        if (tid == 0) out[blockIdx.x] = arg;
        return;
    }
    const float inv_temp = 1.0f / r.temperature;
    const float max_s = max_logit * inv_temp;
    const bool use_p = r.top_p >= 0.f;
    const float top_p = fminf(fmaxf(r.top_p, 0.f), 1.f);

    uint32_t min_key = 0;
    unsigned long long n_keep = (unsigned long long)V;
    if (r.top_k > 0 && r.top_k < V) {
        unsigned long long greater;
        min_key = radix_select<false>(row, V, inv_temp, max_s, 0u, (unsigned long long)r.top_k, sh, &greater);
        // how many reach the threshold (ties included)
        if (tid == 0) sh.count = 0;
        __syncthreads();
        int mine = 0;
        for_each_strided(row, V, tid, [&](int, float v) { mine += key_of(v * inv_temp) >= min_key; });
        mine = (int)rb::warp_sum((float)mine);  // counts are small integers: exact in float
        if (lane == 0) atomicAdd(&sh.count, mine);
        __syncthreads();
        n_keep = (unsigned long long)sh.count;
        __syncthreads();
    }

    if (r.top_k > 0 && n_keep <= (unsigned long long)MAX_CAND) {
        // ---- route 1: candidates in shared memory ----------------------------------------------
        if (tid == 0) sh.count = 0;
        sh.cand_val[tid] = -INFINITY;
        sh.cand_idx[tid] = 0x7fffffff;
        __syncthreads();
        for_each_strided(row, V, tid, [&](int i, float v) {
            const float s = v * inv_temp;
            if (key_of(s) >= min_key) {
                const int pos = atomicAdd(&sh.count, 1);
                sh.cand_val[pos] = s;
                sh.cand_idx[pos] = i;
            }
        });
        __syncthreads();
        const int n = sh.count;
        // bitonic sort of MAX_CAND entries, one per thread; empty entries sort last
        for (int size = 2; size <= MAX_CAND; size <<= 1) {
            for (int stride = size >> 1; stride > 0; stride >>= 1) {
                const int partner = tid ^ stride;
                if (partner > tid) {
                    const bool up = (tid & size) == 0;
                    const float va = sh.cand_val[tid], vb = sh.cand_val[partner];
                    const int ia = sh.cand_idx[tid], ib = sh.cand_idx[partner];
                    const bool a_first = cand_before(va, ia, vb, ib, use_p);
                    if (a_first != up) {
                        sh.cand_val[tid] = vb; sh.cand_val[partner] = va;
                        sh.cand_idx[tid] = ib; sh.cand_idx[partner] = ia;
                    }
                }
                __syncthreads();
            }
        }
        if (tid == 0) {
            float sum = 0.f;
            for (int j = 0; j < n; ++j) { sh.cand_p[j] = expf(sh.cand_val[j] - max_s); sum += sh.cand_p[j]; }
            if (sum > 0.f) for (int j = 0; j < n; ++j) sh.cand_p[j] /= sum;
            int keep = n;
            float eff = 0.f;
            if (use_p) {
                float cum = 0.f;
                for (int j = 0; j < n; ++j) {
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
            out[blockIdx.x] = pick;
        }
        return;
    }

    // ---- route 2: thresholds by radix selection over the whole row ------------------------------
    // total mass of the kept candidates
    unsigned long long part = 0;
    for_each_strided(row, V, tid, [&](int, float v) {
        const float s = v * inv_temp;
        if (key_of(s) >= min_key) part += fixed_of(expf(s - max_s));
    });
    if (tid == 0) sh.acc = 0;
    __syncthreads();
    atomicAdd(&sh.acc, part);
    __syncthreads();
    unsigned long long eff = sh.acc;   // >= 2^40: the maximum itself has probability weight 1
    __syncthreads();
    if (use_p) {
        unsigned long long target = (unsigned long long)((double)top_p * (double)eff);
        target = target < 1 ? 1 : (target > eff ? eff : target);
        unsigned long long greater;
        const uint32_t tp = radix_select<true>(row, V, inv_temp, max_s, min_key, target, sh, &greater);
        min_key = tp > min_key ? tp : min_key;
        // candidates that tie with the threshold enter one by one, in index order, until the
        // cumulative mass reaches the target
        const unsigned long long q = fixed_of(expf(value_of_key(tp) - max_s));
        const unsigned long long ties = q ? (target - greater + q - 1) / q : 1;
        eff = greater + ties * q;
    }
    unsigned long long thr = (unsigned long long)((double)r.u * (double)eff);
    thr = thr < 1 ? 1 : (thr > eff ? eff : thr);
    int token;
    if (use_p) {
        // walk in descending order: the value at which the mass from the top reaches thr, then the
        // j-th candidate of that value in index order
        unsigned long long greater;
        const uint32_t td = radix_select<true>(row, V, inv_temp, max_s, min_key, thr, sh, &greater);
        const unsigned long long q = fixed_of(expf(value_of_key(td) - max_s));
        const unsigned long long j = q ? (thr - greater + q - 1) / q : 1;
        token = index_walk<1>(row, V, inv_temp, max_s, td, j < 1 ? 1 : j, sh, arg);
    } else {
        token = index_walk<0>(row, V, inv_temp, max_s, min_key, thr, sh, arg);
    }
    if (tid == 0) out[blockIdx.x] = token;
}
}  // namespace

// rows: [n] records of 8 x 4 bytes {temperature, top_k, top_p (<0 off), u, penalty (<=0 off),
// hist_begin, hist_len, 0}; history: int32 ids.  logits are modified in place by the penalty.
extern "C" int rb_sample(float* logits, long long row_stride, int n, int V, const void* rows, const int* history,
                         int* out, void* stream) {
    if (n <= 0) return RB_OK;
    if (V <= 0) return RB_ERR_BAD_SIZE;
    RB_LAUNCH((sample_kernel), dim3(n), dim3(ST), 0, (cudaStream_t)stream, logits, row_stride, V, (const SampleRow*)rows, history, out);
    RB_LAUNCH_CHECK();
    return RB_OK;
}
