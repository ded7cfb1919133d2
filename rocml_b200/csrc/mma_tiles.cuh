// Pieces shared by the tensor-core attention kernels: cp.async copies into shared-memory tiles whose
// 16-byte chunks are XOR-swizzled by the row number (so that ldmatrix is free of bank conflicts),
// ldmatrix, and the bfloat16 mma.sync with float32 accumulation.
#pragma once
#include "common.cuh"

namespace mma_tiles {
using namespace rb;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool pred) {
    const int n = pred ? 16 : 0;   // 0: nothing is read, the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// A tile of `rows` rows of HD bf16 in shared memory; row r, 16-byte chunk c lives at chunk c ^ (r & 7).
template <int HD>
__device__ __forceinline__ uint32_t tile_addr(uint32_t base, int row, int chunk) {
    return base + (uint32_t)(row * (HD * 2) + ((chunk ^ (row & 7)) << 4));
}

// Copy `rows` x HD bf16 from global rows (stride in elements) into a swizzled tile; rows >= valid
// are zero-filled.
template <int HD>
__device__ __forceinline__ void load_tile(__nv_bfloat16* tile, const __nv_bfloat16* src, long long stride,
                                          int rows, int valid, int tid, int nthreads) {
    constexpr int CH = HD / 8;
    for (int idx = tid; idx < rows * CH; idx += nthreads) {
        const int r = idx / CH, c = idx % CH;
        const bool ok = r < valid;
        const __nv_bfloat16* g = src + (ok ? (long long)r * stride + c * 8 : 0);
        cp_async16(reinterpret_cast<uint8_t*>(tile) + r * (HD * 2) + ((c ^ (r & 7)) << 4), g, ok);
    }
}

}  // namespace mma_tiles
