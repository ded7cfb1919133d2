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
}  // namespace

extern "C" int rb_argmax(const float* logits, long long row_stride, int rows, int V, int* out, void* stream) {
    if (rows <= 0) return RB_OK;
    if (V <= 0) return RB_ERR_BAD_SIZE;
    argmax_kernel<<<rows, 1024, 0, (cudaStream_t)stream>>>(logits, row_stride, V, out);
    RB_LAUNCH_CHECK();
    return RB_OK;
}
