// Ops-level gated delta rule: the sequential recurrence over T tokens, plus its two elementwise companions.
//
//   gdn_recurrent_kernel  <- the packed recurrence kernel of the reference, qwen35/gated_delta.py:33-137
//                            (per token: S <- g S; kv = S k; d = (v - kv) beta; S <- S + d k^T; y = S q; fp32 state)
//   gdn_gates_kernel      <- compute_g (qwen35/gated_delta.py:16-18) and beta = sigmoid(b) (:158) with the bf16 rounding
//                            points of the reference (qwen35/mslib.py:11-26)
//   gdn_normalize_qk_kernel <- normalize_qk (qwen35/gated_delta.py:21-30)
//
// The recurrence is serial in T, so the only parallelism is (batch, head, value row): one block owns 16 value rows of one
// head, a row is spread over 8 lanes (16 fp32 state values per thread, kept in registers for the whole sequence), and the
// next token's q/k/v/g/beta are fetched while the current one is being applied.
#include "gdn_common.cuh"
#include "launchers.cuh"

namespace gdn {


struct TokenRegs {
    uint2 k[4], q[4];
    float v, g, beta;
};

__global__ void __launch_bounds__(128) gdn_recurrent_kernel(const RecurrentArgs a) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, sub = lane >> 3, l8 = lane & 7;
    const int nsl = a.Dv / 16;
    const int blk = blockIdx.x;
    const int b = blk / (a.Hv * nsl), hv = (blk / nsl) % a.Hv, slice = blk % nsl;
    const int hk = hv / (a.Hv / a.Hk);
    const int row = slice * 16 + warp * 4 + sub;
    const size_t n = (size_t)b * a.Hv + hv;

    float4 s[4];
    if (a.state_in) {
        const float* rp = a.state_in + (n * a.Dv + row) * DK + l8 * 4;
#pragma unroll
        for (int i = 0; i < 4; i++) s[i] = *reinterpret_cast<const float4*>(rp + 32 * i);
    } else {
#pragma unroll
        for (int i = 0; i < 4; i++) s[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }

    const __nv_bfloat16* qp = a.q + ((size_t)b * a.T * a.Hk + hk) * DK + l8 * 4;
    const __nv_bfloat16* kp = a.k + ((size_t)b * a.T * a.Hk + hk) * DK + l8 * 4;
    const __nv_bfloat16* vp = a.v + ((size_t)b * a.T * a.Hv + hv) * a.Dv + row;
    __nv_bfloat16* yp = a.y + ((size_t)b * a.T * a.Hv + hv) * a.Dv + row;
    const float* gp = a.g + (size_t)b * a.T * a.Hv + hv;
    const float* bp = a.beta + (size_t)b * a.T * a.Hv + hv;

    auto fetch = [&](int t, TokenRegs& r) {
        const size_t o = (size_t)t * a.Hk * DK;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            r.k[i] = *reinterpret_cast<const uint2*>(kp + o + 32 * i);
            r.q[i] = *reinterpret_cast<const uint2*>(qp + o + 32 * i);
        }
        r.v = ldbf(vp + (size_t)t * a.Hv * a.Dv);
        r.g = gp[(size_t)t * a.Hv];
        r.beta = bp[(size_t)t * a.Hv];
    };

    TokenRegs cur, nxt;
    if (a.T > 0) fetch(0, cur);
    for (int t = 0; t < a.T; t++) {
        if (t + 1 < a.T) fetch(t + 1, nxt);
        float kvm = 0.f;
        float kf[4][4], qf[4][4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            unpack_bf16x4(cur.k[i], kf[i]);
            unpack_bf16x4(cur.q[i], qf[i]);
            s[i].x *= cur.g; s[i].y *= cur.g; s[i].z *= cur.g; s[i].w *= cur.g;
            kvm += (s[i].x * kf[i][0] + s[i].y * kf[i][1]) + (s[i].z * kf[i][2] + s[i].w * kf[i][3]);
        }
        kvm += __shfl_xor_sync(0xffffffffu, kvm, 1);
        kvm += __shfl_xor_sync(0xffffffffu, kvm, 2);
        kvm += __shfl_xor_sync(0xffffffffu, kvm, 4);
        const float delta = (cur.v - kvm) * cur.beta;
        float yv = 0.f;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            s[i].x += kf[i][0] * delta; s[i].y += kf[i][1] * delta; s[i].z += kf[i][2] * delta; s[i].w += kf[i][3] * delta;
            yv += (s[i].x * qf[i][0] + s[i].y * qf[i][1]) + (s[i].z * qf[i][2] + s[i].w * qf[i][3]);
        }
        yv += __shfl_xor_sync(0xffffffffu, yv, 1);
        yv += __shfl_xor_sync(0xffffffffu, yv, 2);
        yv += __shfl_xor_sync(0xffffffffu, yv, 4);
        if (l8 == 0) yp[(size_t)t * a.Hv * a.Dv] = __float2bfloat16_rn(yv);
        cur = nxt;
    }
    float* op = a.state_out + (n * a.Dv + row) * DK + l8 * 4;
#pragma unroll
    for (int i = 0; i < 4; i++) *reinterpret_cast<float4*>(op + 32 * i) = s[i];
}

int launch_recurrent(const RecurrentArgs& a, cudaStream_t stream) {
    if (a.B <= 0 || a.Hv <= 0) return GDN_OK;
    gdn_recurrent_kernel<<<a.B * a.Hv * (a.Dv / 16), 128, 0, stream>>>(a);
    return check_launch("gdn_recurrent");
}

// ----------------------------------------------------------------------------------------------------------------------
// gates: one thread per (row, head).  a, b are bf16 with an arbitrary row stride (they are columns of the in_proj output).
// ----------------------------------------------------------------------------------------------------------------------
__global__ void gdn_gates_kernel(const __nv_bfloat16* a, const __nv_bfloat16* b, long long a_stride, long long b_stride,
                                 const float* A_log, const float* dt_bias, float* g, float* lg, float* beta, long long n_rows, int H) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_rows * H) return;
    const long long r = i / H;
    const int h = (int)(i % H);
    if (a) {
        const float l = log_decay(expf(A_log[h]), ldbf(a + r * a_stride + h), dt_bias[h]);
        if (lg) lg[i] = l;
        if (g) g[i] = expf(l);
    }
    if (b && beta) beta[i] = sigmoid_bf16(ldbf(b + r * b_stride + h));
}

int launch_gates(const __nv_bfloat16* a, const __nv_bfloat16* b, long long a_stride, long long b_stride, const float* A_log,
                 const float* dt_bias, float* g, float* lg, float* beta, long long n_rows, int H, cudaStream_t stream) {
    const long long n = n_rows * H;
    if (n <= 0) return GDN_OK;
    gdn_gates_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(a, b, a_stride, b_stride, A_log, dt_bias, g, lg, beta, n_rows, H);
    return check_launch("gdn_gates");
}

// ----------------------------------------------------------------------------------------------------------------------
// q/k l2norm: one warp per 128-wide row; out = bf16(bf16(x * rsqrt(mean(x^2) + eps*inv_scale^2)) * bf16(scale))
// ----------------------------------------------------------------------------------------------------------------------
__global__ void gdn_normalize_qk_kernel(const __nv_bfloat16* q, const __nv_bfloat16* k, __nv_bfloat16* qo, __nv_bfloat16* ko,
                                        long long n_rows, float inv_scale, float eps) {
    const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (w >= 2 * n_rows) return;
    const bool is_k = w >= n_rows;
    const long long r = is_k ? w - n_rows : w;
    const __nv_bfloat16* src = (is_k ? k : q) + r * DK + lane * 4;
    __nv_bfloat16* dst = (is_k ? ko : qo) + r * DK + lane * 4;
    float f[4];
    unpack_bf16x4(*reinterpret_cast<const uint2*>(src), f);
    const float ss = warp_sum((f[0] * f[0] + f[1] * f[1]) + (f[2] * f[2] + f[3] * f[3]));
    const float rr = 1.0f / sqrtf(ss / (float)DK + eps * inv_scale * inv_scale);
    const float sc = is_k ? bf(inv_scale) : bf(inv_scale * inv_scale);
    uint2 o;
    o.x = pack_bf16x2(bf(f[0] * rr) * sc, bf(f[1] * rr) * sc);
    o.y = pack_bf16x2(bf(f[2] * rr) * sc, bf(f[3] * rr) * sc);
    *reinterpret_cast<uint2*>(dst) = o;
}

int launch_normalize_qk(const __nv_bfloat16* q, const __nv_bfloat16* k, __nv_bfloat16* qo, __nv_bfloat16* ko, long long n_rows,
                        float inv_scale, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return GDN_OK;
    const long long threads = 2 * n_rows * 32;
    gdn_normalize_qk_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(q, k, qo, ko, n_rows, inv_scale, eps);
    return check_launch("gdn_normalize_qk");
}

}  // namespace gdn
