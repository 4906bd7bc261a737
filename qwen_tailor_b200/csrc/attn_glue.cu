// Elementwise glue around the two attention kernels.
//
//   gqa_qkv_prep_kernel   <- the MLX library calls between the qkv projection and the attention of a full-attention layer
//                            (qwen35/fast.py:70-78 = qwen35/batch.py:504-511 = qwen35/model.py:148-161): split the row into
//                            q | gate per head, k, v; rms_norm(q, q_norm), rms_norm(k, k_norm); RoPE on the first 64 of
//                            256 dims (half-split pairing, base 1e7) at the row's position
//   gqa_gate_out_kernel   <- o * sigmoid(gate) (qwen35/fast.py:84, qwen35/batch.py:512)
//   gdn_conv_prep_kernel  <- conv(4 taps) + silu + q/k l2norm of the prefill path (qwen35/prefill.py:96-134,160-238) and the
//                            new conv window = last 3 raw rows (qwen35/prefill.py:262-263)
//   gdn_gated_norm_kernel <- silu(z) * rmsnorm(y) * w on the GDN output (qwen35/prefill.py:137-157)
// All four are bound by streaming their rows once; bf16 rounding points follow the reference (one rounding per MLX op).
#include "gdn_common.cuh"
#include "launchers.cuh"

namespace gdn {

constexpr int AH = 8, AKV = 2, AD = 256, ROPE = 64;

// one warp per (row, slot); slots 0-7 = q heads, 8-9 = k heads, 10-11 = v heads; lane l owns elements l, l+32, ..., l+224
__global__ void gqa_qkv_prep_kernel(const __nv_bfloat16* qkv, long long row_stride, const float* q_norm, const float* k_norm,
                                    const int* row_pos, __nv_bfloat16* q, __nv_bfloat16* gate, __nv_bfloat16* k, __nv_bfloat16* v,
                                    int R, float eps, float log2_theta) {
    const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (w >= R * 12) return;
    const int r = w / 12, slot = w % 12;
    const __nv_bfloat16* row = qkv + (size_t)r * row_stride;
    if (slot >= 10) {                                            // v: plain copy
        const int kv = slot - 10;
#pragma unroll
        for (int e = 0; e < 8; e++) v[((size_t)r * AKV + kv) * AD + lane + 32 * e] = row[AH * 2 * AD + AKV * AD + kv * AD + lane + 32 * e];
        return;
    }
    const bool is_q = slot < 8;
    const __nv_bfloat16* src = is_q ? row + slot * 2 * AD : row + AH * 2 * AD + (slot - 8) * AD;
    const float* nw = is_q ? q_norm : k_norm;
    float x[8], ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; e++) { x[e] = ldbf(src + lane + 32 * e); ss += x[e] * x[e]; }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)AD + eps);
#pragma unroll
    for (int e = 0; e < 8; e++) x[e] = bf(x[e] * inv * nw[lane + 32 * e]);          // mx.fast.rms_norm: fp32 inside, one rounding
    // RoPE, non-traditional: element i < 32 pairs with i + 32; angle = pos * theta^(-i / 32)
    const float pos = (float)row_pos[r];
    const float ang = pos * exp2f(-(float)lane * (log2_theta / (float)(ROPE / 2)));
    float sn, cs;
    sincosf(ang, &sn, &cs);
    const float x1 = x[0], x2 = x[1];
    x[0] = bf(x1 * cs - x2 * sn);
    x[1] = bf(x1 * sn + x2 * cs);
    __nv_bfloat16* dst = is_q ? q + ((size_t)r * AH + slot) * AD : k + ((size_t)r * AKV + (slot - 8)) * AD;
#pragma unroll
    for (int e = 0; e < 8; e++) dst[lane + 32 * e] = __float2bfloat16_rn(x[e]);
    if (is_q) {
#pragma unroll
        for (int e = 0; e < 8; e++) gate[((size_t)r * AH + slot) * AD + lane + 32 * e] = src[AD + lane + 32 * e];
    }
}

__global__ void gqa_gate_out_kernel(const __nv_bfloat16* o, const __nv_bfloat16* gate, __nv_bfloat16* out, long long n) {
    const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= n) return;
    float a[4], g[4];
    unpack_bf16x4(*reinterpret_cast<const uint2*>(o + i), a);
    unpack_bf16x4(*reinterpret_cast<const uint2*>(gate + i), g);
    uint2 r;
    r.x = pack_bf16x2(a[0] * sigmoid_bf16(g[0]), a[1] * sigmoid_bf16(g[1]));
    r.y = pack_bf16x2(a[2] * sigmoid_bf16(g[2]), a[3] * sigmoid_bf16(g[3]));
    *reinterpret_cast<uint2*>(out + i) = r;
}

// one warp per (token, head, part) with part 0 = q, 1 = k, 2 = v; lane owns 4 consecutive channels
__global__ void gdn_conv_prep_kernel(const __nv_bfloat16* proj, long long row_stride, const __nv_bfloat16* conv_state, const __nv_bfloat16* conv_w,
                                     __nv_bfloat16* q, __nv_bfloat16* k, __nv_bfloat16* v, __nv_bfloat16* new_conv, int S) {
    const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (w >= (long long)S * HV * 3) return;
    const int t = (int)(w / (HV * 3)), hv = (int)((w / 3) % HV), part = (int)(w % 3);
    const int ch = part * KD + hv * DK + lane * 4;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int tap = 0; tap < 4; tap++) {
        const int tt = t - 3 + tap;                                  // rows before the sequence come from the stored window
        const __nv_bfloat16* src = tt < 0 ? conv_state + (size_t)(tt + 3) * CD + ch : proj + (size_t)tt * row_stride + ch;
        float x[4];
        unpack_bf16x4(*reinterpret_cast<const uint2*>(src), x);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float wv = ldbf(conv_w + (size_t)(ch + i) * 4 + tap);
            acc[i] = tap == 0 ? x[i] * wv : acc[i] + x[i] * wv;
        }
    }
    float o[4], ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; i++) { o[i] = silu_bf16(bf(acc[i])); ss += o[i] * o[i]; }
    __nv_bfloat16* dst = (part == 0 ? q : part == 1 ? k : v) + ((size_t)t * HV + hv) * DK + lane * 4;
    if (part < 2) {
        ss = warp_sum(ss);
        const float inv_scale = 0.08838834764831845f;
        const float rr = 1.0f / sqrtf(ss / (float)DK + 1e-6f * inv_scale * inv_scale);
        const float sc = part == 0 ? bf(inv_scale * inv_scale) : bf(inv_scale);
#pragma unroll
        for (int i = 0; i < 4; i++) o[i] = bf(o[i] * rr) * sc;
    }
    uint2 pk;
    pk.x = pack_bf16x2(o[0], o[1]);
    pk.y = pack_bf16x2(o[2], o[3]);
    *reinterpret_cast<uint2*>(dst) = pk;
    if (t >= S - 3) {                                                // new window = last 3 raw rows (older rows come from the old window)
        const int slot = t - (S - 3);
        *reinterpret_cast<uint2*>(new_conv + (size_t)slot * CD + ch) = *reinterpret_cast<const uint2*>(proj + (size_t)t * row_stride + ch);
    }
    if (S < 3 && t == 0) {                                           // short sequences keep the tail of the old window
        for (int slot = 0; slot < 3 - S; slot++)
            *reinterpret_cast<uint2*>(new_conv + (size_t)slot * CD + ch) = *reinterpret_cast<const uint2*>(conv_state + (size_t)(slot + S) * CD + ch);
    }
}

// one warp per (token, head): out = bf16(silu(z) * w * (y * rsqrt(mean(y^2) + 1e-6)))
__global__ void gdn_gated_norm_kernel(const __nv_bfloat16* y, const __nv_bfloat16* proj, long long row_stride, const float* gw, __nv_bfloat16* out,
                                      long long S) {
    const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (w >= S * HV) return;
    const long long t = w / HV;
    const int hv = (int)(w % HV), c0 = lane * 4;
    float yy[4], zz[4];
    unpack_bf16x4(*reinterpret_cast<const uint2*>(y + (size_t)t * (HV * DV) + hv * DV + c0), yy);
    unpack_bf16x4(*reinterpret_cast<const uint2*>(proj + (size_t)t * row_stride + CD + hv * DV + c0), zz);
    float ss = gnorm_sq4(yy);
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);      // neighbouring groups first (see gnorm_sq4)
    const float inv = gnorm_inv(ss);
    float r[4];
#pragma unroll
    for (int i = 0; i < 4; i++) r[i] = gnorm_elem(zz[i], yy[i], inv, gw[c0 + i]);
    uint2 pk;
    pk.x = pack_bf16x2(r[0], r[1]);
    pk.y = pack_bf16x2(r[2], r[3]);
    *reinterpret_cast<uint2*>(out + (size_t)t * (HV * DV) + hv * DV + c0) = pk;
}

int launch_qkv_prep(const __nv_bfloat16* qkv, long long row_stride, const float* q_norm, const float* k_norm, const int* row_pos, __nv_bfloat16* q,
                    __nv_bfloat16* gate, __nv_bfloat16* k, __nv_bfloat16* v, int R, float eps, float theta, cudaStream_t st) {
    if (R <= 0) return GDN_OK;
    const long long threads = (long long)R * 12 * 32;
    gqa_qkv_prep_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(qkv, row_stride, q_norm, k_norm, row_pos, q, gate, k, v, R, eps, log2f(theta));
    return check_launch("gqa_qkv_prep");
}
int launch_gate_out(const __nv_bfloat16* o, const __nv_bfloat16* gate, __nv_bfloat16* out, long long n, cudaStream_t st) {
    if (n <= 0) return GDN_OK;
    gqa_gate_out_kernel<<<(unsigned)((n / 4 + 255) / 256), 256, 0, st>>>(o, gate, out, n);
    return check_launch("gqa_gate_out");
}
int launch_conv_prep(const __nv_bfloat16* proj, long long row_stride, const __nv_bfloat16* conv_state, const __nv_bfloat16* conv_w, __nv_bfloat16* q,
                     __nv_bfloat16* k, __nv_bfloat16* v, __nv_bfloat16* new_conv, int S, cudaStream_t st) {
    if (S <= 0) return GDN_OK;
    const long long threads = (long long)S * HV * 3 * 32;
    gdn_conv_prep_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(proj, row_stride, conv_state, conv_w, q, k, v, new_conv, S);
    return check_launch("gdn_conv_prep");
}
int launch_gated_norm(const __nv_bfloat16* y, const __nv_bfloat16* proj, long long row_stride, const float* gw, __nv_bfloat16* out, long long S,
                      cudaStream_t st) {
    if (S <= 0) return GDN_OK;
    const long long threads = S * HV * 32;
    gdn_gated_norm_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(y, proj, row_stride, gw, out, S);
    return check_launch("gdn_gated_norm");
}

}  // namespace gdn
