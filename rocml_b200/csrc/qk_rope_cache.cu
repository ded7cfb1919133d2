// Fused per-head RMSNorm of q and k, rotary position encoding, and the write of k and v into
// the paged cache.
//
// One warp per (token, head).  Input row layout: [q heads | k heads | v heads], each head
// `hd` wide.  q is normalised and rotated in place; k is normalised, rotated and stored at
// its page; v is stored as it is.  Takes the place of 2x rmsnorm_f32, 2x rope_neox_f32 and
// scatter_kv_chunk / cast_f32_f16 of the reference (rocml/src/forward/attention_chunk.rs:
// 128-197); order as there: norm, then rotation, then the cache write, all before attention.
//
// Rotation (rocml-kernels/kernels/rope.hip:18-33): for i < rot/2, a = pos * inv_freq[i],
// (x_i, x_{i+rot/2}) <- (x_i cos a - x_{i+rot/2} sin a, x_i sin a + x_{i+rot/2} cos a).
// inv_freq comes from the position-encoding part, so another encoding only changes the table.
#include "common.cuh"
#include "api.h"

using namespace rb;

// `in` holds the projections: [S][T, row_stride] of type IT, S partial sums added first, in order
// (S = 1 and IT = AT when the matrix product wrote its result in one piece).  q goes to q_out
// (which may be `in` itself when S = 1 and the types agree), k and v to the cache.
template <typename IT, typename AT, typename WT>
__global__ void qk_norm_rope_cache_kernel(const IT* __restrict__ in, int n_in, size_t in_stride, int row_stride,
                                          AT* __restrict__ q_out, int q_stride, int T, int nq, int nkv, int hd,
                                          const WT* __restrict__ q_norm_w, const WT* __restrict__ k_norm_w,
                                          float eps, const float* __restrict__ inv_freq, int rot_dim,
                                          const int* __restrict__ positions,
                                          const int* __restrict__ slot_of_token,
                                          const int* __restrict__ block_table, int max_pages,
                                          AT* __restrict__ k_cache, AT* __restrict__ v_cache, int write_kv,
                                          const float2* __restrict__ cs_table) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    const int warps_per_block = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* buf = smem + (size_t)warp * hd;
    const int heads_total = nq + (write_kv ? 2 * nkv : 0);
    const long long item = (long long)blockIdx.x * warps_per_block + warp;
    if (item >= (long long)T * heads_total) return;
    const int t = (int)(item / heads_total);
    const int h = (int)(item - (long long)t * heads_total);
    const int slot = slot_of_token[t];
    if (slot < 0) return;  // padding
    const int pos = positions[t];

    int kind, head;  // 0 q, 1 k, 2 v
    if (h < nq) { kind = 0; head = h; }
    else if (h < nq + nkv) { kind = 1; head = h - nq; }
    else { kind = 2; head = h - nq - nkv; }
    const IT* src = in + (size_t)t * row_stride + (size_t)h * hd;

    AT* dst;
    if (kind == 0) {
        dst = q_out + (size_t)t * q_stride + (size_t)head * hd;
    } else {
        const int page = block_table[(size_t)slot * max_pages + (pos / RB_PAGE)];
        if (page < 0) return;  // no page: the host never schedules this; skip rather than fault
        AT* base = (kind == 1 ? k_cache : v_cache);
        dst = base + (((size_t)page * nkv + head) * RB_PAGE + (pos % RB_PAGE)) * hd;
    }

    float ss = 0.f;
    if (n_in > 1 && sizeof(IT) == 4 && (hd & 3) == 0 && (in_stride & 3) == 0 && (row_stride & 3) == 0 &&
        ((uintptr_t)in & 15) == 0) {
        // partial sums in float32: 16-byte loads, four partial sums in flight, added in order
        const float4* s4 = reinterpret_cast<const float4*>(src);
        const size_t st4 = in_stride >> 2;
        for (int i = lane; i < (hd >> 2); i += 32) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            int s = 0;
            for (; s + 4 <= n_in; s += 4) {
                const float4 a = s4[(size_t)s * st4 + i], b = s4[(size_t)(s + 1) * st4 + i];
                const float4 c = s4[(size_t)(s + 2) * st4 + i], d = s4[(size_t)(s + 3) * st4 + i];
                v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
                v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
                v.x += c.x; v.y += c.y; v.z += c.z; v.w += c.w;
                v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
            }
            for (; s < n_in; ++s) {
                const float4 d = s4[(size_t)s * st4 + i];
                v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
            }
            buf[4 * i] = v.x; buf[4 * i + 1] = v.y; buf[4 * i + 2] = v.z; buf[4 * i + 3] = v.w;
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    } else {
        for (int i = lane; i < hd; i += 32) {
            float v = 0.f;
            for (int s = 0; s < n_in; ++s) v += to_f32(src[(size_t)s * in_stride + i]);
            buf[i] = v;
            ss += v * v;
        }
    }
    __syncwarp();
    if (kind == 2) {
        for (int i = lane; i < hd; i += 32) dst[i] = from_f32<AT>(buf[i]);
        return;
    }
    ss = warp_sum(ss);
    const WT* w = kind == 0 ? q_norm_w : k_norm_w;
    const float inv = w ? rsqrtf(ss / (float)hd + eps) : 1.f;
    const int half = inv_freq ? rot_dim / 2 : 0;
    for (int i = lane; i < half; i += 32) {
        float x0 = buf[i], x1 = buf[i + half];
        if (w) { x0 = x0 * inv * to_f32(w[i]); x1 = x1 * inv * to_f32(w[i + half]); }
        float sn, cs;
        if (cs_table) { const float2 c2 = cs_table[(size_t)t * half + i]; cs = c2.x; sn = c2.y; }
        else sincosf((float)pos * inv_freq[i], &sn, &cs);
        dst[i] = from_f32<AT>(x0 * cs - x1 * sn);
        dst[i + half] = from_f32<AT>(x0 * sn + x1 * cs);
    }
    for (int i = 2 * half + lane; i < hd; i += 32) {
        float x = buf[i];
        if (w) x = x * inv * to_f32(w[i]);
        dst[i] = from_f32<AT>(x);
    }
}

// The same for a head size of 128 with the whole head rotated, the common case: a lane holds 4
// consecutive dimensions (one 8- or 16-byte load per partial sum), the rotation partner sits 16 lanes
// away (shuffle), nothing goes through shared memory, and a head is written with 8-byte stores.
// A warp takes HPW heads of one token: their loads go out together before anything is computed, and
// the token's angles and the norms' weights are loaded once for all of them (16-byte loads).  One
// head a warp left the kernel waiting on a chain of small loads: 30 us for a prompt of 2,048 tokens
// (50 MB, a quarter of the memory's bandwidth).
constexpr int HPW = 4;

template <typename WT>
__device__ __forceinline__ void load_w4(const WT* w, int lane, float* out) {
    if (sizeof(WT) == 4) {
        const float4 f = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w) + lane * 4);
        out[0] = f.x; out[1] = f.y; out[2] = f.z; out[3] = f.w;
    } else {
        const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(w) + lane * 4);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        out[0] = a.x; out[1] = a.y; out[2] = b.x; out[3] = b.y;
    }
}

template <typename IT, typename AT, typename WT>
__global__ void __launch_bounds__(128)
qk_norm_rope_cache_hd128_kernel(const IT* __restrict__ in, int n_in, size_t in_stride, int row_stride,
                                AT* __restrict__ q_out, int q_stride, int T, int nq, int nkv,
                                const WT* __restrict__ q_norm_w, const WT* __restrict__ k_norm_w, float eps,
                                const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                const int* __restrict__ slot_of_token, const int* __restrict__ block_table,
                                int max_pages, AT* __restrict__ k_cache, AT* __restrict__ v_cache, int write_kv,
                                const float2* __restrict__ cs_table) {
    pdl_trigger();
    constexpr int hd = 128;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads_total = nq + (write_kv ? 2 * nkv : 0);
    const int groups = (heads_total + HPW - 1) / HPW;             // groups of heads a token
    const long long item = (long long)blockIdx.x * 4 + warp;
    // the norms' weights do not depend on the kernel before this one
    float wq[4] = {1.f, 1.f, 1.f, 1.f}, wk[4] = {1.f, 1.f, 1.f, 1.f};
    const bool has_w = q_norm_w != nullptr;
    if (has_w) { load_w4(q_norm_w, lane, wq); load_w4(k_norm_w, lane, wk); }
    pdl_wait();
    if (item >= (long long)T * groups) return;
    const int t = (int)(item / groups);
    const int h0 = (int)(item - (long long)t * groups) * HPW;
    const int slot = slot_of_token[t];
    if (slot < 0) return;
    const int pos = positions[t];
    const int n_heads = min(HPW, heads_total - h0);
    const IT* src = in + (size_t)t * row_stride + (size_t)h0 * hd + lane * 4;
    // What depends on the token alone is asked for before the heads' values, so that everything is in flight
    // together: its angles, and the page of its key and value if this warp holds any.
    float4 cs_a = make_float4(1.f, 0.f, 1.f, 0.f), cs_b = cs_a;
    if (inv_freq && cs_table) {
        const float4* c4 = reinterpret_cast<const float4*>(cs_table + (size_t)t * 64 + (lane & 15) * 4);
        cs_a = c4[0];
        cs_b = c4[1];
    }
    int page = -2;
    if (write_kv && h0 + n_heads > nq) page = block_table[(size_t)slot * max_pages + (pos / RB_PAGE)];
    // every head's values: the loads of all heads (and of up to 8 partial sums each) are in flight together
    float v[HPW][4];
#pragma unroll
    for (int j = 0; j < HPW; ++j) { v[j][0] = v[j][1] = v[j][2] = v[j][3] = 0.f; }
    if (sizeof(IT) == 4) {
        for (int s = 0; s < n_in; s += 4) {
            float4 f[HPW][4];
#pragma unroll
            for (int j = 0; j < HPW; ++j)
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    f[j][u] = (j < n_heads && s + u < n_in)
                                  ? *reinterpret_cast<const float4*>(src + (size_t)(s + u) * in_stride + j * hd)
                                  : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int j = 0; j < HPW; ++j)
#pragma unroll
                for (int u = 0; u < 4; ++u) { v[j][0] += f[j][u].x; v[j][1] += f[j][u].y; v[j][2] += f[j][u].z; v[j][3] += f[j][u].w; }
        }
    } else {
        for (int s = 0; s < n_in; ++s) {
            uint2 raw[HPW];
#pragma unroll
            for (int j = 0; j < HPW; ++j)
                raw[j] = j < n_heads ? *reinterpret_cast<const uint2*>(src + (size_t)s * in_stride + j * hd) : make_uint2(0u, 0u);
#pragma unroll
            for (int j = 0; j < HPW; ++j) {
                const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[j].x));
                const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[j].y));
                v[j][0] += a.x; v[j][1] += a.y; v[j][2] += b.x; v[j][3] += b.y;
            }
        }
    }
    // the token's angles, once for all its heads: (cos, sin) of dimensions (lane & 15) * 4 .. + 3
    float cs[4] = {1.f, 1.f, 1.f, 1.f}, sn[4] = {0.f, 0.f, 0.f, 0.f};
    if (inv_freq) {
        if (cs_table) {
            const float4 a = cs_a, b = cs_b;
            cs[0] = a.x; sn[0] = a.y; cs[1] = a.z; sn[1] = a.w; cs[2] = b.x; sn[2] = b.y; cs[3] = b.z; sn[3] = b.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) sincosf((float)pos * inv_freq[(lane & 15) * 4 + j], &sn[j], &cs[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < HPW; ++j) {
        if (j >= n_heads) continue;
        const int h = h0 + j;
        const int kind = h < nq ? 0 : (h < nq + nkv ? 1 : 2);   // 0 q, 1 k, 2 v
        AT* dst;
        if (kind == 0) {
            dst = q_out + (size_t)t * q_stride + (size_t)h * hd;
        } else {
            if (page < 0) continue;                             // no page: the host never schedules this
            const int head = kind == 1 ? h - nq : h - nq - nkv;
            dst = (kind == 1 ? k_cache : v_cache) + (((size_t)page * nkv + head) * RB_PAGE + (pos % RB_PAGE)) * hd;
        }
        float (&x)[4] = v[j];
        if (kind != 2) {
            if (has_w) {
                const float ss = warp_sum(x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3]);
                const float inv = rsqrtf(ss / (float)hd + eps);
#pragma unroll
                for (int i = 0; i < 4; ++i) x[i] = x[i] * inv * (kind == 0 ? wq[i] : wk[i]);
            }
            if (inv_freq) {
                // dimension i < 64 pairs with i + 64: lanes 0-15 hold x_i, lanes 16-31 the partners
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float other = __shfl_xor_sync(0xffffffffu, x[i], 16);
                    x[i] = lane < 16 ? x[i] * cs[i] - other * sn[i] : other * sn[i] + x[i] * cs[i];
                }
            }
        }
        if (sizeof(AT) == 4) {
            *reinterpret_cast<float4*>(dst + lane * 4) = make_float4(x[0], x[1], x[2], x[3]);
        } else {
            __nv_bfloat162 lo = __floats2bfloat162_rn(x[0], x[1]), hi = __floats2bfloat162_rn(x[2], x[3]);
            uint2 raw;
            raw.x = *reinterpret_cast<uint32_t*>(&lo);
            raw.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(dst + lane * 4) = raw;
        }
    }
}

template <typename IT, typename AT, typename WT>
static int launch_qk(const void* in, int n_in, long long in_stride, int row_stride, void* q_out, int q_stride,
                     int T, int nq, int nkv, int hd, const void* qw, const void* kw, float eps,
                     const float* inv_freq, int rot_dim, const int* positions, const int* slot_of_token,
                     const int* block_table, int max_pages, void* k_cache, void* v_cache, int write_kv,
                     const float2* cs_table, cudaStream_t s) {
    const int warps = 4;
    const long long items = (long long)T * (nq + (write_kv ? 2 * nkv : 0));
    const long long blocks = (items + warps - 1) / warps;
    if (blocks > 0x7fffffffLL) return RB_ERR_BAD_SIZE;
    const size_t esz = sizeof(IT);
    if (hd == 128 && (!inv_freq || rot_dim == 128) && (((uintptr_t)in | (uintptr_t)q_out | (uintptr_t)k_cache |
                                                        (uintptr_t)v_cache | (uintptr_t)qw | (uintptr_t)kw |
                                                        (uintptr_t)cs_table) & 15) == 0 &&
        (row_stride * esz) % 16 == 0 && ((size_t)in_stride * esz) % 16 == 0 && (q_stride * sizeof(AT)) % 16 == 0) {
        const long long groups = (long long)T * ((nq + (write_kv ? 2 * nkv : 0) + HPW - 1) / HPW);
        RB_LAUNCH((qk_norm_rope_cache_hd128_kernel<IT, AT, WT>), dim3((int)((groups + 3) / 4)), dim3(128), 0, s, (const IT*)in, n_in,
                  (size_t)in_stride, row_stride, (AT*)q_out, q_stride, T, nq, nkv, (const WT*)qw, (const WT*)kw, eps,
                  inv_freq, positions, slot_of_token, block_table, max_pages, (AT*)k_cache, (AT*)v_cache, write_kv,
                  cs_table);
        return RB_OK;
    }
    const size_t smem = (size_t)warps * hd * sizeof(float);
    if (smem > 48 * 1024) return RB_ERR_BAD_SIZE;
    RB_LAUNCH((qk_norm_rope_cache_kernel<IT, AT, WT>), dim3((int)blocks), dim3(warps * 32), smem, s, (const IT*)in,
              n_in, (size_t)in_stride, row_stride, (AT*)q_out, q_stride, T, nq, nkv, hd, (const WT*)qw,
              (const WT*)kw, eps, inv_freq, rot_dim, positions, slot_of_token, block_table, max_pages,
              (AT*)k_cache, (AT*)v_cache, write_kv, cs_table);
    return RB_OK;
}

extern "C" int rb_qk_norm_rope_cache(const void* in, int in_dtype, int n_in, long long in_stride, int row_stride,
                                     void* q_out, int act_dtype, int q_stride, int T, int nq, int nkv, int hd,
                                     const void* q_norm_w, const void* k_norm_w, int w_dtype, float eps,
                                     const float* inv_freq, int rot_dim, const int* positions,
                                     const int* slot_of_token, const int* block_table, int max_pages,
                                     void* k_cache, void* v_cache, int write_kv, const void* cos_sin, void* stream) {
    if (T <= 0) return RB_OK;
    if (hd <= 0 || hd % 2 || n_in < 1 || (inv_freq && (rot_dim <= 0 || rot_dim % 2 || rot_dim > hd)))
        return RB_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    typedef __nv_bfloat16 bf;
#define RB_QK_ARGS in, n_in, in_stride, row_stride, q_out, q_stride, T, nq, nkv, hd, q_norm_w, k_norm_w, eps, \
                   inv_freq, rot_dim, positions, slot_of_token, block_table, max_pages, k_cache, v_cache, write_kv, \
                   (const float2*)cos_sin, s
    if (in_dtype == RB_BF16 && act_dtype == RB_BF16 && w_dtype == RB_BF16) return launch_qk<bf, bf, bf>(RB_QK_ARGS);
    if (in_dtype == RB_BF16 && act_dtype == RB_BF16 && w_dtype == RB_F32) return launch_qk<bf, bf, float>(RB_QK_ARGS);
    if (in_dtype == RB_F32 && act_dtype == RB_BF16 && w_dtype == RB_BF16) return launch_qk<float, bf, bf>(RB_QK_ARGS);
    if (in_dtype == RB_F32 && act_dtype == RB_BF16 && w_dtype == RB_F32) return launch_qk<float, bf, float>(RB_QK_ARGS);
    if (in_dtype == RB_F32 && act_dtype == RB_F32 && w_dtype == RB_BF16) return launch_qk<float, float, bf>(RB_QK_ARGS);
    if (in_dtype == RB_F32 && act_dtype == RB_F32 && w_dtype == RB_F32) return launch_qk<float, float, float>(RB_QK_ARGS);
#undef RB_QK_ARGS
    return RB_ERR_BAD_DTYPE;
}

// cos and sin of pos * inv_freq[i] for every token of a step, [T][half] pairs (cos, sin): computed
// once per step with full-precision sincosf and read by every layer's rotation.
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq, int T,
                                  int half, float2* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= T * half) return;
    const int t = idx / half, i = idx - t * half;
    float sn, cs;
    sincosf((float)positions[t] * inv_freq[i], &sn, &cs);
    out[idx] = make_float2(cs, sn);
}

extern "C" int rb_rope_table(const int* positions, const float* inv_freq, int T, int half, void* out, void* stream) {
    if (T <= 0 || half <= 0) return RB_OK;
    const long long n = (long long)T * half;
    if (n > 0x7fffffffLL) return RB_ERR_BAD_SIZE;
    RB_LAUNCH((rope_table_kernel), dim3((unsigned)((n + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, positions,
              inv_freq, T, half, (float2*)out);
    return RB_OK;
}
