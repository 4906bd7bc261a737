// GatedDeltaNet recurrent decode / speculative-verify kernel.
//
// One launch runs M chained tokens for each of B sequences: depthwise causal conv (4 taps) + silu on the mixed qkv row,
// q/k l2norm, gates, the gated delta rule on the fp32 [16,128,128] state, and a state + conv-window snapshot after every
// token.  It replaces three Metal kernels of the reference that share this arithmetic and differ only in where the state
// lives: `deltanet` (qwen35/kernels.py:461-567, functional snapshots), `deltanet_b` (qwen35/batch.py:36-135, slot pools
// updated in place) and `deltanet_bm` (qwen35/batch_spec.py:45-150, snapshot pools updated in place).
//
// The kernel is bound by HBM traffic on the state (1 MiB read + M MiB written per sequence and layer).  Mapping:
//   grid  = B x 16 heads x (128 / ROWS) value-row slices, 128 threads per block
//   a state row (128 fp32 = 512 B) is spread over 8 lanes: lane l holds the float4s at columns 4l + 32i, i < 4, so a warp
//   load instruction touches four complete 128-byte lines; the two 128-wide dot products per row are finished with three
//   xor-shuffles inside the 8-lane group.  Each thread keeps its 16 (ROWS=16) or 32 (ROWS=32) state values in registers
//   across the M tokens and streams one snapshot per token back with 128-bit stores.
//   The conv/norm prologue of a token is computed once per block into shared memory (thread t = channel t of q and k).
#include "gdn_common.cuh"
#include "launchers.cuh"

namespace gdn {


template <int PASSES>
__global__ void __launch_bounds__(128) gdn_decode_kernel(const DecodeArgs a) {
    constexpr int ROWS = 16 * PASSES;
    constexpr int NSL = DV / ROWS;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, sub = lane >> 3, l8 = lane & 7;
    const int blk = blockIdx.x;
    const int b = blk / (HV * NSL), hv = (blk / NSL) % HV, slice = blk % NSL;
    const int row_base = slice * ROWS;
    const int M = a.M;

    // ---- where this sequence's state lives (qwen35/kernels.py:473-474, batch.py:47-54, batch_spec.py:57-65) ----
    const __nv_bfloat16* cs_in;
    __nv_bfloat16* cs_out;
    const float* st_in;
    float* st_out;
    {
        const int e = a.i0[a.mode == 0 ? 0 : b];
        if (e < 0 || e >= a.n_entries) { if (tid == 0) atomicExch(a.status, 1); return; }
        if (a.mode == 0) {
            cs_in = a.conv_pool + (size_t)e * 3 * CD;
            cs_out = a.conv_out;
            st_in = a.ssm_pool + (size_t)e * STATE_ELEMS;
            st_out = a.ssm_out;
        } else if (a.mode == 1) {
            const unsigned par = (unsigned)a.i1[b] & 1u;
            cs_in = a.conv_pool + ((size_t)e * 2 + par) * 3 * CD;
            cs_out = a.conv_pool + ((size_t)e * 2 + (par ^ 1u)) * 3 * CD;
            st_in = a.ssm_pool + (size_t)e * STATE_ELEMS;
            st_out = a.ssm_pool + (size_t)e * STATE_ELEMS;
        } else {
            const int sl = a.i1[b];
            if (sl < 0 || sl >= M) { if (tid == 0) atomicExch(a.status, 1); return; }
            const unsigned par = (unsigned)a.i2[b] & 1u;
            cs_in = a.conv_pool + (((size_t)e * 2 + par) * M + sl) * 3 * CD;
            cs_out = a.conv_pool + (((size_t)e * 2 + (par ^ 1u)) * M) * 3 * CD;
            st_out = a.ssm_pool + (size_t)e * M * STATE_ELEMS;
            st_in = st_out + (size_t)sl * STATE_ELEMS;
        }
    }
    const __nv_bfloat16* pj = a.proj + (size_t)b * M * a.row_stride;
    __nv_bfloat16* yb = a.y + (size_t)b * M * (HV * DV);

    __shared__ __align__(16) float sq[DK];
    __shared__ __align__(16) float sk[DK];
    __shared__ float sv[ROWS], sy[ROWS], sred[8];

    // ---- state rows into registers (issued first: everything below overlaps with these loads) ----
    float4 s[PASSES][4];
    int rows[PASSES];
#pragma unroll
    for (int p = 0; p < PASSES; p++) {
        rows[p] = row_base + (warp * PASSES + p) * 4 + sub;
        const float* rp = st_in + ((size_t)hv * DV + rows[p]) * DK + l8 * 4;
#pragma unroll
        for (int i = 0; i < 4; i++) s[p][i] = *reinterpret_cast<const float4*>(rp + 32 * i);
    }

    const float inv_scale = 0.08838834764831845f;          // 128^-1/2
    const float e2 = 1e-6f * inv_scale * inv_scale;
    const float sc_q = bf(inv_scale * inv_scale), sc_k = bf(inv_scale);
    const float expA = expf(a.A_log[hv]);
    const float dtb = a.dt_bias[hv];

    // input row t of channel ch: t < 0 reads the stored window (qwen35/kernels.py:477-479)
    auto inp = [&](int t, int ch) -> float {
        return t < 0 ? ldbf(cs_in + (t + 3) * CD + ch) : ldbf(pj + (size_t)t * a.row_stride + ch);
    };
    auto conv = [&](int j, int ch) -> float {
        const uint2 wb = *reinterpret_cast<const uint2*>(a.conv_w + (size_t)ch * 4);
        float w[4];
        unpack_bf16x4(wb, w);
        float o = inp(j - 3, ch) * w[0];
        o += inp(j - 2, ch) * w[1];
        o += inp(j - 1, ch) * w[2];
        o += inp(j, ch) * w[3];
        return silu_bf16(bf(o));
    };
    auto put_window = [&](int j, int ch) {                 // conv snapshot j = rows j-2, j-1, j (qwen35/kernels.py:528-541)
#pragma unroll
        for (int t = 0; t < 3; t++) cs_out[((size_t)j * 3 + t) * CD + ch] = __float2bfloat16_rn(inp(j - 2 + t, ch));
    };

    for (int j = 0; j < M; j++) {
        // ---- prologue: conv + silu for this head's q / k channels and this block's v rows ----
        const int chq = hv * DK + tid, chk = KD + hv * DK + tid;
        const float qv = conv(j, chq), kv = conv(j, chk);
        const float qs_w = warp_sum(qv * qv), ks_w = warp_sum(kv * kv);
        if (lane == 0) { sred[warp] = qs_w; sred[4 + warp] = ks_w; }
        if (tid < ROWS) {
            const int chv = 2 * KD + hv * DV + row_base + tid;
            sv[tid] = conv(j, chv);
            put_window(j, chv);
        }
        if (slice == 0) { put_window(j, chq); put_window(j, chk); }
        __syncthreads();
        const float qs = (sred[0] + sred[1]) + (sred[2] + sred[3]);
        const float ks = (sred[4] + sred[5]) + (sred[6] + sred[7]);
        const float qr = 1.0f / sqrtf(qs / (float)DK + e2);
        const float kr = 1.0f / sqrtf(ks / (float)DK + e2);
        sq[tid] = bf(bf(qv * qr) * sc_q);                   // l2norm(q) / sqrt(128), rounded like the reference (kernels.py:504-509)
        sk[tid] = bf(bf(kv * kr) * sc_k);
        const float av = ldbf(pj + (size_t)j * a.row_stride + CD + KD + HV + hv);
        const float g = expf(log_decay(expA, av, dtb));
        const float beta = sigmoid_bf16(ldbf(pj + (size_t)j * a.row_stride + CD + KD + hv));
        __syncthreads();

        float4 kk[4], qq[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            kk[i] = *reinterpret_cast<const float4*>(sk + l8 * 4 + 32 * i);
            qq[i] = *reinterpret_cast<const float4*>(sq + l8 * 4 + 32 * i);
        }
        float* so = st_out + (size_t)j * STATE_ELEMS;
#pragma unroll
        for (int p = 0; p < PASSES; p++) {
            float kvm = 0.f;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                s[p][i].x *= g; s[p][i].y *= g; s[p][i].z *= g; s[p][i].w *= g;
                kvm += (s[p][i].x * kk[i].x + s[p][i].y * kk[i].y) + (s[p][i].z * kk[i].z + s[p][i].w * kk[i].w);
            }
            kvm += __shfl_xor_sync(0xffffffffu, kvm, 1);
            kvm += __shfl_xor_sync(0xffffffffu, kvm, 2);
            kvm += __shfl_xor_sync(0xffffffffu, kvm, 4);
            const float delta = (sv[rows[p] - row_base] - kvm) * beta;
            float yv = 0.f;
            float* rp = so + ((size_t)hv * DV + rows[p]) * DK + l8 * 4;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                s[p][i].x += kk[i].x * delta; s[p][i].y += kk[i].y * delta;
                s[p][i].z += kk[i].z * delta; s[p][i].w += kk[i].w * delta;
                yv += (s[p][i].x * qq[i].x + s[p][i].y * qq[i].y) + (s[p][i].z * qq[i].z + s[p][i].w * qq[i].w);
                *reinterpret_cast<float4*>(rp + 32 * i) = s[p][i];
            }
            yv += __shfl_xor_sync(0xffffffffu, yv, 1);
            yv += __shfl_xor_sync(0xffffffffu, yv, 2);
            yv += __shfl_xor_sync(0xffffffffu, yv, 4);
            if (l8 == 0) sy[rows[p] - row_base] = yv;
        }
        __syncthreads();
        if (tid < ROWS) yb[(size_t)j * (HV * DV) + hv * DV + row_base + tid] = __float2bfloat16_rn(sy[tid]);
    }
}

int launch_decode(const DecodeArgs& a, cudaStream_t stream) {
    if (a.B <= 0 || a.M <= 0) return GDN_OK;
    // few sequences: 16-row slices double the block count so that one sequence still covers the GPU
    if (a.B <= 8) gdn_decode_kernel<1><<<a.B * HV * 8, 128, 0, stream>>>(a);
    else          gdn_decode_kernel<2><<<a.B * HV * 4, 128, 0, stream>>>(a);
    return check_launch("gdn_decode");
}

}  // namespace gdn
