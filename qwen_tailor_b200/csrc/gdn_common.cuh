// Shared definitions for the GatedDeltaNet / GQA-decode kernels (sm_100a).
//
// Model constants follow the reference's Cfg (qwen35/model.py:35-60) and its kernel headers (qwen35/kernels.py:466):
// 16 value heads, d_k = d_v = 128, mixed-qkv width 6144 = q 2048 | k 2048 | v 2048, in_proj row 8224 = qkv | z 2048 | b 16 | a 16.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "../../include/gdn_b200.h"

namespace gdn {

constexpr int HV = 16, DK = 128, DV = 128, KD = 2048, CD = 6144, PW = 8224;
constexpr int STATE_ELEMS = HV * DV * DK;        // fp32 elements of one (sequence, layer) state

// error codes (GDN_OK, GDN_E_*) come from the public header

void set_error(const char* fmt, ...);             // stores a thread-local message for gdn_last_error_string()
int check_launch(const char* what);               // cudaGetLastError -> GDN_E_LAUNCH (+ message)

// ------------------------------------------------------------------------------------------------------------------
// bf16 <-> fp32 and the "round after every op" bf16 math of the reference (qwen35/mslib.py:11-26)
// ------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float bf(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ float ldbf(const __nv_bfloat16* p) { return __bfloat162float(*p); }

// mx.sigmoid on bf16: 1 / (1 + exp(|x|)), mirrored for x >= 0, rounding after each op
__device__ __forceinline__ float sigmoid_bf16(float x) {
    float y = bf(1.0f / bf(1.0f + bf(expf(fabsf(x)))));
    return x < 0.0f ? y : bf(1.0f - y);
}
__device__ __forceinline__ float silu_bf16(float x) { return bf(x * sigmoid_bf16(x)); }
// nn.softplus on bf16 = logaddexp(x, 0)
__device__ __forceinline__ float softplus_bf16(float x) {
    return bf(fmaxf(x, 0.0f) + bf(log1pf(bf(expf(-fabsf(x))))));
}
// log-decay of one token/head: -exp(A_log) * softplus_bf16(bf16(a + dt_bias))   (qwen35/kernels.py:511-513)
__device__ __forceinline__ float log_decay(float expA, float a, float dtb) { return -expA * softplus_bf16(bf(a + dtb)); }

__device__ __forceinline__ void unpack_bf16x4(uint2 u, float* f) {
    f[0] = __uint_as_float(u.x << 16); f[1] = __uint_as_float(u.x & 0xffff0000u);
    f[2] = __uint_as_float(u.y << 16); f[3] = __uint_as_float(u.y & 0xffff0000u);
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Optional in-kernel time stamps (builds with -DGDN_TIMING only): block 0 logs clock64() at labelled points into the translation
// unit's own g_tlog, which that unit's gdn_timing_log_* function copies out.
#ifdef GDN_TIMING
static __device__ long long g_tlog[8192];
#ifndef GDN_TBLOCK
#define GDN_TBLOCK 0
#endif
#define GDN_TSTAMP(slot) do { if (blockIdx.x == GDN_TBLOCK && (threadIdx.x & 31) == 0 && (slot) < 8192) g_tlog[(slot)] = clock64(); } while (0)
// per-block stamps on the global nanosecond timer: slot 4096 + 16 * block + k
__device__ __forceinline__ long long gdn_globaltimer() { long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
#define GDN_BSTAMP_ANY(k) do { if (blockIdx.x < 250) g_tlog[4096 + 16 * blockIdx.x + (k)] = gdn_globaltimer(); } while (0)
#define GDN_BVAL(k, v) do { if (threadIdx.x == 0 && blockIdx.x < 250) g_tlog[4096 + 16 * blockIdx.x + (k)] = (long long)(v); } while (0)
#define GDN_BSTAMP(k) do { if (threadIdx.x == 0 && blockIdx.x < 250) g_tlog[4096 + 16 * blockIdx.x + (k)] = gdn_globaltimer(); } while (0)
#else
#define GDN_TSTAMP(slot) do { } while (0)
#define GDN_BSTAMP(k) do { } while (0)
#define GDN_BVAL(k, v) do { } while (0)
#define GDN_BSTAMP_ANY(k) do { } while (0)
#endif

// The gated RMSNorm of the GDN output (qwen35/prefill.py:137-157): out = silu(z) * (w * (y * inv)), inv = rsqrt(mean(y^2) + 1e-6).
// One definition for the stand-alone kernel and for the fused y store of the prefill kernel, so that both give the same bits:
// the 128 squares of a row are summed as (y0^2 + y1^2) + (y2^2 + y3^2) per group of four, then pairwise over neighbouring groups
// (group g with g ^ 1, then ^ 2, ^ 4, ^ 8, ^ 16).  exp, the division and rsqrt use the fast hardware approximations (a few fp32 ulp,
// far below the bf16 rounding of the result).
__device__ __forceinline__ float gnorm_sq4(const float* y) { return (y[0] * y[0] + y[1] * y[1]) + (y[2] * y[2] + y[3] * y[3]); }
__device__ __forceinline__ float gnorm_inv(float ss) { return rsqrtf(fmaf(ss, 1.f / 128.f, 1e-6f)); }
__device__ __forceinline__ float gnorm_elem(float z, float y, float inv, float w) {
    return __fmul_rn(__fdividef(z, 1.f + __expf(-z)), __fmul_rn(w, __fmul_rn(y, inv)));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

}  // namespace gdn
