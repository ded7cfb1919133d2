// Shared helpers of the kernels: element types, conversions, reductions, launch checks.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

// Element type codes of the C interface.
#define RB_F32 0
#define RB_BF16 1

// Return codes of the C interface beyond cudaError_t values (which are returned as they are).
#define RB_OK 0
#define RB_ERR_BAD_SIZE 10001      // a size the kernel does not take
#define RB_ERR_BAD_DTYPE 10002     // an element type combination that is not built
#define RB_ERR_BAD_ALIGN 10003     // a pointer or stride that breaks an alignment rule
#define RB_ERR_TIMEOUT 10004       // a bounded wait inside a kernel ran out
#define RB_ERR_NO_DRIVER_FN 10005  // a driver entry point could not be found
#define RB_ERR_IO 10006            // a file could not be read

#define RB_PAGE 64  // tokens per cache page

#define RB_LAUNCH_CHECK()                         \
    do {                                          \
        cudaError_t e__ = cudaGetLastError();     \
        if (e__ != cudaSuccess) return (int)e__;  \
    } while (0)
#define RB_LAUNCH(...)                                       \
    do {                                                     \
        cudaError_t e__ = rb::launch(__VA_ARGS__);           \
        if (e__ != cudaSuccess) return (int)e__;             \
    } while (0)

namespace rb {

// ---- programmatic dependent launch ------------------------------------------------------------
// Every kernel of the library is launched so that it may be scheduled while its predecessor in the
// stream is still running: it signals at once that its own successor may be scheduled
// (pdl_trigger), does whatever does not depend on the predecessor (set-up, and for the matrix
// products the first tiles of the weights), and only then waits for the predecessor's results
// (pdl_wait, which returns once the predecessor has finished and its writes are visible).  Without
// the launch attribute both instructions do nothing.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool pdl_enabled();  // defined in launch.cu: on unless RB_PDL=0 is set

template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// The same with the grid's blocks grouped into clusters (every grid extent a multiple of the cluster's):
// the blocks of a cluster run at the same time and can read and write each other's shared memory.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_clustered(void (*kernel)(KArgs...), dim3 grid, dim3 block, dim3 cluster, size_t smem,
                                    cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster.x;
    attr[0].val.clusterDim.y = cluster.y;
    attr[0].val.clusterDim.z = cluster.z;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();  // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

}  // namespace rb
