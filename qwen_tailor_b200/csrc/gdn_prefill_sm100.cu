// Chunked GatedDeltaNet prefill on the Blackwell tensor cores (tcgen05 / TMEM / TMA), chunk size 64, varlen batches.
//
// Replaces the reference's two-phase chunked kernel `gdn_chunked` (qwen35/gdn_nax.py:413-426; phase A :71-143, phase B
// :224-358), which works on 16-token chunks with Apple simdgroup MMAs.  Same algebra (qwen35/gdn_nax.py:3-10), per head and
// chunk of C = 64 tokens, S0 = state entering the chunk ([dv, dk]), Lc = inclusive cumulative log-decay in the chunk:
//     L  = strict_lower(beta_i exp(Lc_i - Lc_j) (K K^T)_ij)        T = (I + L)^-1,  Tb = T diag(beta)
//     D  = Tb (V - gamma * (K S0^T))                               gamma_i = exp(Lc_i)
//     Y  = gamma * (Q S0^T) + A D,  A = lower_incl(exp(Lc_i - Lc_j) (Q K^T)_ij)
//     S1 = gamma_C S0 + D^T diag(exp(Lc_C - Lc_j)) K
// Decay factors are always exp of a masked difference of Lc (never a ratio), so the ~1e-97 in-chunk decays of real gates
// underflow to 0 instead of producing inf * 0.
//
// Mapping.  One block = one (sequence, head) chain; the chain over chunks is serial, heads / sequences / layers are the
// parallel axis.  Every product is computed TRANSPOSED so that the 128 value rows of the head are the M dimension of a
// full-rate M = 128 MMA and the TMEM lane of a thread is "its" value row for the whole kernel:
//     G    [128 x 64]  = [K; Q] K^T          rows 0-63 = K K^T, rows 64-127 = Q K^T (K and Q tiles are stacked in smem)
//     P1^T [dv x 64]   = S0 K^T,  P2^T = S0 Q^T                       A = S0 (bf16 hi + lo) from TMEM
//     D^T  [dv x 64]   = Z^T Tb^T,  Z^T = V^T - P1^T diag(gamma)      A = Z^T (hi + lo) from TMEM, B = Tb (hi + lo) in smem
//     AD^T [dv x 64]   = D^T A^T                                      A = D^T (hi + lo) from TMEM, B = A (hi + lo) in smem
//     S    [dv x 128] += Dp^T K,  Dp = diag(dec) D                    A = Dp^T (hi + lo) in smem, B = K read MN-major
// The fp32 state lives in TMEM for the whole sequence.  Every operand that is derived from fp32 data (S, Z, D, Dp, Tb, A) is
// fed to the bf16 MMA as an exact hi + lo pair (16 significand bits), which keeps the final state within 1e-4 of fp64; K, Q
// and V are bf16 already.  (I + L)^-1 is an exact fp32 forward substitution (one column per thread), as in the reference
// (qwen35/gdn_nax.py:118-141): the tensor-core products with T are the "solve products".
// K/Q/V chunks arrive by TMA (128-byte swizzle, no multicast), double buffered; rows of a partial last chunk are zeroed in
// shared memory so that a packed neighbour sequence can never leak in.
#include <cuda.h>
#include "gdn_common.cuh"
#include "launchers.cuh"
#include "sm100_prims.cuh"

namespace gdn {

using namespace sm100;

constexpr int CH = 64;                               // chunk length
// ---- shared memory map (bytes from a 1024-aligned base) ----
constexpr int SM_STAGE = 48 * 1024;                  // per stage: [K_h0 | Q_h0 | K_h1 | Q_h1] (4 x 8 KiB) + [V_h0 | V_h1] (2 x 8 KiB)
constexpr int SM_V = 32 * 1024;                      // offset of V inside a stage
constexpr int SM_TB_HI = 2 * SM_STAGE;               // Tb hi / lo, A hi / lo: [64][64] bf16, K-major, 8 KiB each
constexpr int SM_TB_LO = SM_TB_HI + 8192;
constexpr int SM_A_HI = SM_TB_LO + 8192;
constexpr int SM_A_LO = SM_A_HI + 8192;
constexpr int SM_DP_HI = SM_A_LO + 8192;             // Dp^T hi / lo: [128][64] bf16, K-major, 16 KiB each
constexpr int SM_DP_LO = SM_DP_HI + 16384;
constexpr int SM_L = SM_DP_LO + 16384;               // L fp32 [64][LSTRIDE]
constexpr int LSTRIDE = 68;
constexpr int SM_GATES = SM_L + 64 * LSTRIDE * 4;    // Lc, gamma, dec, beta [64] fp32 each + scratch
constexpr int SM_TOTAL = SM_GATES + 5 * 256 + 64;
// ---- tensor memory map (columns) ----
constexpr uint32_t TM_S = 0;                         // fp32 state, pre-scaled by the coming chunk's gamma_C   [128 cols]
constexpr uint32_t TM_SHI = 128, TM_SLO = 192;       // bf16 pairs of the unscaled state                        [64 + 64]
constexpr uint32_t TM_G = 256;                       // [K;Q] K^T, later A D                                    [64]
constexpr uint32_t TM_P1 = 320;                      // S0 K^T, later D^T                                       [64]
constexpr uint32_t TM_P2 = 384;                      // S0 Q^T                                                  [64]
constexpr uint32_t TM_ZHI = 448, TM_ZLO = 480;       // Z^T, later D^T, as bf16 pairs                           [32 + 32]

__device__ __forceinline__ void split_pack(float x0, float x1, uint32_t& hi, uint32_t& lo) {
    const float h0 = bf(x0), h1 = bf(x1);
    hi = pack_bf16x2(h0, h1);
    lo = pack_bf16x2(x0 - h0, x1 - h1);
}

// exact forward substitution for column j of T = (I + L)^-1, rows I0..63 (rows above I0 are zero for columns >= I0)
template <int I0>
__device__ __forceinline__ void solve_column(const float* Lm, int j, float (&x)[64]) {
#pragma unroll
    for (int i = 0; i < I0; i++) x[i] = 0.f;
#pragma unroll
    for (int i = I0; i < 64; i++) {
        float acc = (i == j) ? 1.f : 0.f;
#pragma unroll
        for (int m4 = I0; m4 < i; m4 += 4) {
            const float4 l = *reinterpret_cast<const float4*>(Lm + i * LSTRIDE + m4);
            acc -= l.x * x[m4];
            if (m4 + 1 < i) acc -= l.y * x[m4 + 1];
            if (m4 + 2 < i) acc -= l.z * x[m4 + 2];
            if (m4 + 3 < i) acc -= l.w * x[m4 + 3];
        }
        x[i] = acc;
    }
}

__global__ void __launch_bounds__(128, 1)
gdn_prefill_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                   const PrefillArgs a) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t bars[3];
    __shared__ uint32_t tmem_slot;
    __shared__ float s_red[8];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int seq = blockIdx.x / a.n_heads, h = a.head_lo + blockIdx.x % a.n_heads;
    const int t_begin = a.cu_seqlens[seq], t_end = a.cu_seqlens[seq + 1];
    const int len = t_end - t_begin;
    float* fin = a.final_state + ((size_t)seq * a.H + h) * DV * DK + (size_t)tid * DK;
    const float* init = nullptr;
    if (a.init_state) {
        const int ii = a.init_idx ? a.init_idx[seq] : seq;
        if (ii >= 0) init = a.init_state + ((size_t)ii * a.H + h) * DV * DK + (size_t)tid * DK;
    }
    if (len <= 0 || t_begin < 0 || t_end > a.total_T) {
        // nothing to compute: the state passes through unchanged
        if (len < 0 || t_begin < 0 || t_end > a.total_T) { if (tid == 0) atomicExch(a.status, 1); return; }
        for (int c = 0; c < DK; c += 4)
            *reinterpret_cast<float4*>(fin + c) = init ? *reinterpret_cast<const float4*>(init + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        return;
    }
    const int nchunks = (len + CH - 1) / CH;

    const uint32_t sbase = smem_addr(smem);
    const uint32_t bar_tma0 = smem_addr(&bars[0]), bar_tma1 = smem_addr(&bars[1]), bar_mma = smem_addr(&bars[2]);
    float* Lm = reinterpret_cast<float*>(smem + SM_L);
    float* s_Lc = reinterpret_cast<float*>(smem + SM_GATES);
    float* s_gam = s_Lc + 64;
    float* s_dec = s_gam + 64;
    float* s_beta = s_dec + 64;

    if (tid == 0) {
        mbar_init(bar_tma0, 1); mbar_init(bar_tma1, 1); mbar_init(bar_mma, 1);
        fence_barrier_init();
        tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
    }
    if (warp == 0) { tmem_alloc(smem_addr(&tmem_slot), 512); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tb = tmem_slot;
    const uint32_t tl = tb + ((uint32_t)(warp * 32) << 16);          // this warp's 32 lanes

    auto issue_tma = [&](int c) {                                    // thread 0: K, Q, V of chunk c -> stage c & 1
        const uint32_t st = sbase + (c & 1) * SM_STAGE;
        const uint32_t bar = (c & 1) ? bar_tma1 : bar_tma0;
        const int t0 = t_begin + c * CH;
        mbar_expect_tx(bar, 6 * 8192);
        tma_load_3d(st, &tmK, bar, 0, h, t0);
        tma_load_3d(st + 8192, &tmQ, bar, 0, h, t0);
        tma_load_3d(st + 16384, &tmK, bar, 64, h, t0);
        tma_load_3d(st + 24576, &tmQ, bar, 64, h, t0);
        tma_load_3d(st + SM_V, &tmV, bar, 0, h, t0);
        tma_load_3d(st + SM_V + 8192, &tmV, bar, 64, h, t0);
    };
    if (tid == 0) issue_tma(0);

    // total log-decay of a chunk (threads 0..63 each take one row); every thread gets the result
    auto chunk_log_decay = [&](int c) -> float {
        float x = 0.f;
        const int t = t_begin + c * CH + tid;
        if (tid < 64 && c < nchunks && t < t_end) x = a.lg[(size_t)t * a.H + h];
        x = warp_sum(x);
        __syncthreads();
        if (lane == 0) s_red[warp] = x;
        __syncthreads();
        return s_red[0] + s_red[1];
    };

    // ---- initial state -> TMEM: unscaled bf16 hi/lo pairs and the fp32 copy pre-scaled by gamma_C of chunk 0 ----
    float gC_cur = expf(chunk_log_decay(0));
    for (int blk = 0; blk < 4; blk++) {
        uint32_t r[32], hi[16], lo[16];
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
            const float4 v4 = init ? *reinterpret_cast<const float4*>(init + blk * 32 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            split_pack(v4.x, v4.y, hi[i / 2], lo[i / 2]);
            split_pack(v4.z, v4.w, hi[i / 2 + 1], lo[i / 2 + 1]);
            r[i] = __float_as_uint(v4.x * gC_cur); r[i + 1] = __float_as_uint(v4.y * gC_cur);
            r[i + 2] = __float_as_uint(v4.z * gC_cur); r[i + 3] = __float_as_uint(v4.w * gC_cur);
        }
        tmem_st32(tl + TM_S + blk * 32, r);
        tmem_st16(tl + TM_SHI + blk * 16, hi);
        tmem_st16(tl + TM_SLO + blk * 16, lo);
    }
    tmem_wait_st();

    constexpr uint32_t I64 = idesc_bf16(128, 64, 0, 0);              // N = 64, both operands K-major
    constexpr uint32_t I128MN = idesc_bf16(128, 128, 0, 1);          // N = 128, B read MN-major
    uint32_t mma_phase = 0;
    bool ok = true;

    for (int c = 0; c < nchunks; c++) {
        const int stage = c & 1;
        const uint32_t st = sbase + stage * SM_STAGE;
        const int t0 = t_begin + c * CH;
        const int nrows = min(CH, t_end - t0);
        const bool last = c == nchunks - 1;

        // ---- gates of this chunk: Lc (inclusive prefix sum of the log-decay), gamma, dec, beta; total decay of the next chunk ----
        float lgj = 0.f, bj = 0.f, lgn = 0.f;
        if (tid < 64) {
            if (tid < nrows) { lgj = a.lg[(size_t)(t0 + tid) * a.H + h]; bj = a.beta[(size_t)(t0 + tid) * a.H + h]; }
            if (!last && t0 + CH + tid < t_end) lgn = a.lg[(size_t)(t0 + CH + tid) * a.H + h];
        }
        float xs = lgj;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const float y = __shfl_up_sync(0xffffffffu, xs, o); if (lane >= o) xs += y; }
        const float nsum = warp_sum(lgn);
        if (lane == 31) s_red[warp] = xs;
        if (lane == 0) s_red[4 + warp] = nsum;
        __syncthreads();
        if (warp == 1) xs += s_red[0];
        const float Ltot = s_red[0] + s_red[1];
        const float gC_next = expf(s_red[4] + s_red[5]);
        if (tid < 64) { s_Lc[tid] = xs; s_gam[tid] = expf(xs); s_dec[tid] = expf(Ltot - xs); s_beta[tid] = bj; }

        // ---- this chunk's tiles have landed; start the next chunk's copy into the other stage ----
        ok &= mbar_wait(stage ? bar_tma1 : bar_tma0, (uint32_t)(c >> 1) & 1u);
        if (tid == 0 && !last) issue_tma(c + 1);
        if (nrows < CH) {
            // rows past the end of the sequence are zero (qwen35/gdn_nax.py:55-60): 6 tiles x (64 - nrows) rows x 128 B
            const int nz = (CH - nrows) * 8;                          // 16-byte pieces per tile
            for (int i = tid; i < 6 * nz; i += 128) {
                const int tile = i / nz, p = i % nz;
                *reinterpret_cast<uint4*>(smem + stage * SM_STAGE + tile * 8192 + nrows * 128 + p * 16) = make_uint4(0, 0, 0, 0);
            }
            fence_proxy_async_smem();
        }
        tc_fence_before_sync();
        if (!__syncthreads_and(ok)) break;

        // ---- G = [K; Q] K^T ----
        if (tid == 0) {
            tc_fence_after_sync();
#pragma unroll
            for (int ks = 0; ks < 8; ks++) {
                const uint32_t off = (ks >> 2) * 16384 + (ks & 3) * 32;
                mma_ss(tb + TM_G, smem_desc_sw128(st + off, 16, 1024), smem_desc_sw128(st + off, 16, 1024), I64, ks > 0);
            }
            mma_commit(bar_mma);
        }
        ok &= mbar_wait(bar_mma, mma_phase); mma_phase ^= 1;
        tc_fence_after_sync();

        // ---- L (threads 0..63, fp32 to smem) and A (threads 64..127, bf16 hi/lo K-major rows) from G ----
        {
            const int i = tid & 63;
            const float Li = s_Lc[i], bi = s_beta[i];
#pragma unroll
            for (int half = 0; half < 2; half++) {
                uint32_t r[32];
                tmem_ld32(tl + TM_G + half * 32, r);
                tmem_wait_ld();
                if (tid < 64) {
#pragma unroll
                    for (int jj = 0; jj < 32; jj += 4) {
                        float4 o;
                        float* op = &o.x;
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const int j = half * 32 + jj + e;
                            op[e] = (j < i) ? bi * expf(Li - s_Lc[j]) * __uint_as_float(r[jj + e]) : 0.f;
                        }
                        *reinterpret_cast<float4*>(Lm + i * LSTRIDE + half * 32 + jj) = o;
                    }
                } else {
#pragma unroll
                    for (int cb = 0; cb < 4; cb++) {                  // 16-byte pieces: 8 columns each
                        uint32_t hi[4], lo[4];
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const int j = half * 32 + cb * 8 + 2 * e;
                            const float a0 = (j <= i) ? expf(Li - s_Lc[j]) * __uint_as_float(r[cb * 8 + 2 * e]) : 0.f;
                            const float a1 = (j + 1 <= i) ? expf(Li - s_Lc[j + 1]) * __uint_as_float(r[cb * 8 + 2 * e + 1]) : 0.f;
                            split_pack(a0, a1, hi[e], lo[e]);
                        }
                        const uint32_t o = i * 128 + (((half * 4 + cb) ^ (i & 7)) << 4);
                        *reinterpret_cast<uint4*>(smem + SM_A_HI + o) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                        *reinterpret_cast<uint4*>(smem + SM_A_LO + o) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                    }
                }
            }
        }
        __syncthreads();

        // ---- T = (I + L)^-1 by forward substitution, one column per thread; Tb = T diag(beta) as bf16 hi/lo, K-major rows ----
        if (tid < 64) {
            float x[64];
            if (warp == 0) solve_column<0>(Lm, tid, x); else solve_column<32>(Lm, tid, x);
            const float bj2 = s_beta[tid];
            const uint32_t cpiece = (uint32_t)(tid >> 3), cin = (uint32_t)(tid & 7) * 2;
#pragma unroll
            for (int i = 0; i < 64; i++) {
                const float tv = x[i] * bj2;
                const float hi = bf(tv);
                const uint32_t o = i * 128 + ((cpiece ^ (i & 7)) << 4) + cin;
                *reinterpret_cast<__nv_bfloat16*>(smem + SM_TB_HI + o) = __float2bfloat16_rn(hi);
                *reinterpret_cast<__nv_bfloat16*>(smem + SM_TB_LO + o) = __float2bfloat16_rn(tv - hi);
            }
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncthreads();

        // ---- P1^T = S0 K^T, P2^T = S0 Q^T (S0 = hi + lo from TMEM) ----
        if (tid == 0) {
            tc_fence_after_sync();
#pragma unroll
            for (int part = 0; part < 2; part++) {
                const uint32_t acol = part ? TM_SLO : TM_SHI;
#pragma unroll
                for (int ks = 0; ks < 8; ks++) {
                    const uint32_t off = (ks >> 2) * 16384 + (ks & 3) * 32;
                    mma_ts(tb + TM_P1, tb + acol + ks * 8, smem_desc_sw128(st + off, 16, 1024), I64, (part | ks) != 0);
                }
            }
            mma_commit(bar_mma);
#pragma unroll
            for (int part = 0; part < 2; part++) {
                const uint32_t acol = part ? TM_SLO : TM_SHI;
#pragma unroll
                for (int ks = 0; ks < 8; ks++) {
                    const uint32_t off = 8192 + (ks >> 2) * 16384 + (ks & 3) * 32;
                    mma_ts(tb + TM_P2, tb + acol + ks * 8, smem_desc_sw128(st + off, 16, 1024), I64, (part | ks) != 0);
                }
            }
        }
        ok &= mbar_wait(bar_mma, mma_phase); mma_phase ^= 1;
        tc_fence_after_sync();

        // ---- Z^T = V^T - P1^T diag(gamma) -> bf16 hi/lo pairs in TMEM ----
        {
            const unsigned char* vt = smem + stage * SM_STAGE + SM_V + (tid >> 6) * 8192;
            const int vc = tid & 63;
            const uint32_t vpiece = (uint32_t)(vc >> 3), vin = (uint32_t)(vc & 7) * 2;
#pragma unroll
            for (int half = 0; half < 2; half++) {
                uint32_t r[32], hi[16], lo[16];
                tmem_ld32(tl + TM_P1 + half * 32, r);
                tmem_wait_ld();
#pragma unroll
                for (int jj = 0; jj < 32; jj += 2) {
                    const int j = half * 32 + jj;
                    const float v0 = ldbf(reinterpret_cast<const __nv_bfloat16*>(vt + j * 128 + ((vpiece ^ (j & 7)) << 4) + vin));
                    const float v1 = ldbf(reinterpret_cast<const __nv_bfloat16*>(vt + (j + 1) * 128 + ((vpiece ^ ((j + 1) & 7)) << 4) + vin));
                    const float z0 = v0 - s_gam[j] * __uint_as_float(r[jj]);
                    const float z1 = v1 - s_gam[j + 1] * __uint_as_float(r[jj + 1]);
                    split_pack(z0, z1, hi[jj / 2], lo[jj / 2]);
                }
                tmem_st16(tl + TM_ZHI + half * 16, hi);
                tmem_st16(tl + TM_ZLO + half * 16, lo);
            }
            tmem_wait_st();
        }
        tc_fence_before_sync();
        if (!__syncthreads_and(ok)) break;

        // ---- D^T = Z^T Tb^T  (hi*hi + lo*hi + hi*lo) ----
        if (tid == 0) {
            tc_fence_after_sync();
#pragma unroll
            for (int term = 0; term < 3; term++) {
                const uint32_t acol = term == 1 ? TM_ZLO : TM_ZHI;
                const uint32_t bsm = sbase + (term == 2 ? SM_TB_LO : SM_TB_HI);
#pragma unroll
                for (int ks = 0; ks < 4; ks++)
                    mma_ts(tb + TM_P1, tb + acol + ks * 8, smem_desc_sw128(bsm + ks * 32, 16, 1024), I64, (term | ks) != 0);
            }
            mma_commit(bar_mma);
        }
        ok &= mbar_wait(bar_mma, mma_phase); mma_phase ^= 1;
        tc_fence_after_sync();

        // ---- D^T -> bf16 hi/lo pairs in TMEM (A operand of A D) and Dp^T = D^T diag(dec) -> hi/lo K-major rows in smem ----
        {
#pragma unroll
            for (int half = 0; half < 2; half++) {
                uint32_t r[32], hi[16], lo[16];
                tmem_ld32(tl + TM_P1 + half * 32, r);
                tmem_wait_ld();
#pragma unroll
                for (int jj = 0; jj < 32; jj += 2) split_pack(__uint_as_float(r[jj]), __uint_as_float(r[jj + 1]), hi[jj / 2], lo[jj / 2]);
                tmem_st16(tl + TM_ZHI + half * 16, hi);
                tmem_st16(tl + TM_ZLO + half * 16, lo);
#pragma unroll
                for (int cb = 0; cb < 4; cb++) {
                    uint32_t ph[4], pl[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const int jj = cb * 8 + 2 * e, j = half * 32 + jj;
                        split_pack(__uint_as_float(r[jj]) * s_dec[j], __uint_as_float(r[jj + 1]) * s_dec[j + 1], ph[e], pl[e]);
                    }
                    const uint32_t o = tid * 128 + (((half * 4 + cb) ^ (tid & 7)) << 4);
                    *reinterpret_cast<uint4*>(smem + SM_DP_HI + o) = make_uint4(ph[0], ph[1], ph[2], ph[3]);
                    *reinterpret_cast<uint4*>(smem + SM_DP_LO + o) = make_uint4(pl[0], pl[1], pl[2], pl[3]);
                }
            }
            tmem_wait_st();
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        if (!__syncthreads_and(ok)) break;

        // ---- A D (into the G columns) and the state update S += Dp^T K ----
        if (tid == 0) {
            tc_fence_after_sync();
#pragma unroll
            for (int term = 0; term < 3; term++) {
                const uint32_t acol = term == 1 ? TM_ZLO : TM_ZHI;
                const uint32_t bsm = sbase + (term == 2 ? SM_A_LO : SM_A_HI);
#pragma unroll
                for (int ks = 0; ks < 4; ks++)
                    mma_ts(tb + TM_G, tb + acol + ks * 8, smem_desc_sw128(bsm + ks * 32, 16, 1024), I64, (term | ks) != 0);
            }
#pragma unroll
            for (int part = 0; part < 2; part++) {
                const uint32_t asm_ = sbase + (part ? SM_DP_LO : SM_DP_HI);
#pragma unroll
                for (int ks = 0; ks < 4; ks++)
                    mma_ss(tb + TM_S, smem_desc_sw128(asm_ + ks * 32, 16, 1024), smem_desc_sw128(st + ks * 2048, 16384, 1024), I128MN, 1);
            }
            mma_commit(bar_mma);
        }
        ok &= mbar_wait(bar_mma, mma_phase); mma_phase ^= 1;
        tc_fence_after_sync();

        // ---- Y^T = P2^T diag(gamma) + A D  ->  y[t0 + i, h, v]  (thread v = value row) ----
        {
            __nv_bfloat16* yp = a.y + ((size_t)t0 * a.H + h) * DV + tid;
#pragma unroll
            for (int half = 0; half < 2; half++) {
                uint32_t p2[32], ad[32];
                tmem_ld32(tl + TM_P2 + half * 32, p2);
                tmem_ld32(tl + TM_G + half * 32, ad);
                tmem_wait_ld();
#pragma unroll
                for (int ii = 0; ii < 32; ii++) {
                    const int i = half * 32 + ii;
                    if (i < nrows) yp[(size_t)i * a.H * DV] = __float2bfloat16_rn(s_gam[i] * __uint_as_float(p2[ii]) + __uint_as_float(ad[ii]));
                }
            }
        }
        // ---- new state: bf16 hi/lo pairs for the next chunk's products, fp32 copy pre-scaled by the next gamma_C (or the output) ----
        for (int blk = 0; blk < 4; blk++) {
            uint32_t r[32], hi[16], lo[16];
            tmem_ld32(tl + TM_S + blk * 32, r);
            tmem_wait_ld();
            if (last) {
#pragma unroll
                for (int i = 0; i < 32; i += 4)
                    *reinterpret_cast<float4*>(fin + blk * 32 + i) = make_float4(__uint_as_float(r[i]), __uint_as_float(r[i + 1]), __uint_as_float(r[i + 2]),
                                                                               __uint_as_float(r[i + 3]));
            } else {
#pragma unroll
                for (int i = 0; i < 32; i += 2) split_pack(__uint_as_float(r[i]), __uint_as_float(r[i + 1]), hi[i / 2], lo[i / 2]);
#pragma unroll
                for (int i = 0; i < 32; i++) r[i] = __float_as_uint(__uint_as_float(r[i]) * gC_next);
                tmem_st16(tl + TM_SHI + blk * 16, hi);
                tmem_st16(tl + TM_SLO + blk * 16, lo);
                tmem_st32(tl + TM_S + blk * 32, r);
            }
        }
        tmem_wait_st();
        gC_cur = gC_next;
        tc_fence_before_sync();
        if (!__syncthreads_and(ok)) break;
    }
    if (!ok && tid == 0) atomicExch(a.status, 3);                    // a bounded wait gave up
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tb, 512);
}

// ----------------------------------------------------------------------------------------------------------------------
// host side: tensor maps + launch
// ----------------------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        cudaDriverEntryPointQueryResult qr;
        void* p = nullptr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess && qr == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        else
            cudaGetLastError();
    }
    return fn;
}

// [total_T, H, 128] bf16 viewed as a 3-D tensor (128, H, total_T); box = 64 columns x 1 head x 64 tokens, 128-byte swizzle;
// tokens beyond total_T read as zero
static int make_map(CUtensorMap* m, const void* base, long long total_T, int H) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) { set_error("gdn_prefill_chunked: cuTensorMapEncodeTiled is not available from this driver"); return GDN_E_UNSUPPORTED; }
    const cuuint64_t dims[3] = {128, (cuuint64_t)H, (cuuint64_t)total_T};
    const cuuint64_t strides[2] = {256, (cuuint64_t)H * 256};
    const cuuint32_t box[3] = {64, 1, 64}, es[3] = {1, 1, 1};
    const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("gdn_prefill_chunked: cuTensorMapEncodeTiled failed with code %d", (int)r); return GDN_E_LAUNCH; }
    return GDN_OK;
}

int launch_prefill(const void* q, const void* k, const void* v, const PrefillArgs& a, cudaStream_t stream) {
    if (a.n_seq <= 0 || a.n_heads <= 0) return GDN_OK;
    CUtensorMap tq, tk, tv;
    int rc;
    if ((rc = make_map(&tq, q, a.total_T, a.H)) || (rc = make_map(&tk, k, a.total_T, a.H)) || (rc = make_map(&tv, v, a.total_T, a.H))) return rc;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    const int smem = SM_TOTAL + 1024;
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        if (cudaFuncSetAttribute(gdn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return check_launch("gdn_prefill smem attribute");
        attr_set[dev] = true;
    }
    gdn_prefill_kernel<<<a.n_seq * a.n_heads, 128, smem, stream>>>(tq, tk, tv, a);
    return check_launch("gdn_prefill");
}

}  // namespace gdn
