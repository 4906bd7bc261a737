// Phase A of the chunked GatedDeltaNet prefill: everything of a 64-token chunk that does not depend on the recurrent state.
//
// Replaces the reference's phase-A kernels `gdn_nax_a` (qwen35/gdn_nax.py:71-143) and, in the fused flavour, `gdn_nax_prep_a`
// (qwen35/gdn_nax.py:150-222): per (chunk, head), from K, the log-decay and beta of the chunk's tokens,
//     Lc    = inclusive cumulative log2-decay inside the chunk          gamma_i = 2^Lc_i,  dec_i = 2^(Lc_C - Lc_i)
//     L     = strict_lower(beta_i 2^(Lc_i - Lc_j) (K K^T)_ij)
//     T     = (I + L)^-1,   Tb = T diag(beta)
// One block per (chunk, head): every tile of a launch is independent, so a single sequence already fills the GPU (the serial part
// of the prefill is the chain kernel in gdn_prefill_sm100.cu, which reads what this kernel writes).
//
// K K^T runs on the tensor cores (tcgen05.mma, fp32 accumulator in tensor memory, K fetched by one TMA tile load).  The inverse is
// fp32 throughout: exact forward substitution on the four 16 x 16 diagonal blocks (one warp each, a 15-deep dependent chain
// instead of 63), then the off-diagonal blocks are assembled as block products  T_ba = -T_bb (L_ba T_aa)  -- two 16^3 product
// pairs and one 32^3 pair -- on the tensor cores as well (mma.sync tf32, every fp32 operand as a two-term tf32 split with the three
// significant partial products accumulated in fp32, so the products carry fp32-class accuracy).  The reference does the same
// substitution per 16-token chunk (qwen35/gdn_nax.py:118-141); the products of inverse blocks are what a 64-token chunk adds.
//
// Output record of a tile (17,152 bytes, consumed by the chain kernel with one bulk copy):
//     Tb as bf16 hi / lo parts, each a [64][64] K-major operand image with the 128-byte swizzle already applied  (2 x 8 KiB)
//     Lc[64], gamma[64], dec[64] fp32
// Record of chunk c of sequence s, head h:  ((cu_seqlens[s] / 64 + s + c) * H + h).  The slot number cu_seqlens[s] / 64 + s + c is
// unique per (sequence, chunk) and below total_T / 64 + n_seq, so the host can size the buffer without reading cu_seqlens.
//
// Fused flavour (FUSED = true): the block first computes q, k, v of its tile from the in_proj rows -- depthwise causal conv
// (4 taps, sliding window in registers) + silu, q / k l2norm, gates from the a / b columns -- writes them out for the chain kernel
// and keeps k in shared memory, so q / k / v never make a round trip through device memory before phase A.
#include <cuda.h>
#include <cstring>
#include "gdn_common.cuh"
#include "launchers.cuh"
#include "sm100_prims.cuh"

namespace gdn {

using namespace sm100;

constexpr int PA_THREADS = 128;
constexpr int PA_CH = 64;
constexpr int PA_LS = 68;                                  // row stride (floats) of the fp32 L and T tiles
constexpr int PA_SM_K = 0;                                 // K tile: two [64][64] bf16 boxes, 128-byte swizzle (16 KiB); once K K^T
constexpr int PA_SM_T = 0;                                 //   has been formed the same bytes hold T fp32 [64][68]
constexpr int PA_SM_L = 64 * PA_LS * 4;                    // raw K K^T, then L, fp32 [64][68]; consumed blocks take the inner block products
constexpr int PA_SM_G = 2 * 64 * PA_LS * 4;                // Lc[64], beta[64]
constexpr int PA_SM_TOTAL = PA_SM_G + 512;
constexpr uint32_t PA_WAIT_LIMIT = 200000u;

__device__ __forceinline__ float pa_ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }

__device__ __forceinline__ void pa_split_pack(float x0, float x1, uint32_t& hi, uint32_t& lo) {
    hi = pack_bf16x2(x0, x1);
    lo = pack_bf16x2(x0 - __uint_as_float(hi << 16), x1 - __uint_as_float(hi & 0xffff0000u));
}

// bounded wait with a pause between polls
__device__ __forceinline__ bool pa_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < PA_WAIT_LIMIT; i++) {
        if (mbar_test_wait(bar, parity)) return true;
        __nanosleep(40);
    }
    return false;
}

// ---- fp32 block products on the tensor cores: mma.sync m16n8k8 tf32 with each fp32 operand split into two tf32 terms and the
//      three significant partial products accumulated in fp32 (hi hi + lo hi + hi lo: ~21 significand bits, fp32-class accuracy) ----
// hi = x truncated to tf32 (a mask, so the conversion unit stays free for the ex2 of the L build), lo = the exact residual, again
// truncated: hi + lo carries 21 significand bits of x
__device__ __forceinline__ void tf32_split(float x, uint32_t& hi, uint32_t& lo) {
    hi = __float_as_uint(x) & 0xFFFFE000u;
    lo = __float_as_uint(x - __uint_as_float(hi)) & 0xFFFFE000u;
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
// acc[nt] (+)= A[16 x 8 KS] B[8 KS x 8 NT] for one warp: A, B row-major fp32 in shared memory (element (r, c) at p[r * ld + c]),
// A = rows [0, 16), B columns [8 nt, 8 nt + 8).  Fragment layout of m16n8k8: g = lane / 4, t = lane % 4;
// a = {(g, t), (g + 8, t), (g, t + 4), (g + 8, t + 4)}, b = {(t, g), (t + 4, g)}, c = {(g, 2t), (g, 2t + 1), (g + 8, 2t), (g + 8, 2t + 1)}.
template <int KS, int NT>
__device__ __forceinline__ void warp_mm_tf32x3(const float* __restrict__ A, int lda, const float* __restrict__ B, int ldb, int lane, float (&acc)[NT][4]) {
    const int g = lane >> 2, t = lane & 3;
    float lo1[NT][4], lo2[NT][4];                                     // the two small partial products keep their own accumulators:
#pragma unroll                                                        // three independent MMA chains instead of one three times as long
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int e = 0; e < 4; e++) { lo1[nt][e] = 0.f; lo2[nt][e] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < KS; ks++) {
        uint32_t ah[4], al[4];
        tf32_split(A[g * lda + 8 * ks + t], ah[0], al[0]);
        tf32_split(A[(g + 8) * lda + 8 * ks + t], ah[1], al[1]);
        tf32_split(A[g * lda + 8 * ks + t + 4], ah[2], al[2]);
        tf32_split(A[(g + 8) * lda + 8 * ks + t + 4], ah[3], al[3]);
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            uint32_t bh[2], bl[2];
            tf32_split(B[(8 * ks + t) * ldb + 8 * nt + g], bh[0], bl[0]);
            tf32_split(B[(8 * ks + t + 4) * ldb + 8 * nt + g], bh[1], bl[1]);
            mma_tf32(lo1[nt], al, bh);
            mma_tf32(lo2[nt], ah, bl);
            mma_tf32(acc[nt], ah, bh);
        }
    }
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int e = 0; e < 4; e++) acc[nt][e] += lo1[nt][e] + lo2[nt][e];
}

// (sequence, chunk) of a record slot: slot = cu_seqlens[s] / 64 + s + c.  Returns false for slots that no chunk maps to.
__device__ __forceinline__ bool slot_to_chunk(const int* __restrict__ cu, int n_seq, int slot, int& seq, int& c) {
    int lo = 0, hi = n_seq - 1;
    while (lo < hi) {
        const int m = (lo + hi + 1) >> 1;
        if (cu[m] / PA_CH + m <= slot) lo = m; else hi = m - 1;
    }
    seq = lo;
    c = slot - (cu[lo] / PA_CH + lo);
    const int len = cu[lo + 1] - cu[lo];
    return c >= 0 && c < (len + PA_CH - 1) / PA_CH;
}

template <bool FUSED>
__global__ void __launch_bounds__(PA_THREADS, 6)
gdn_phase_a_kernel(const __grid_constant__ CUtensorMap tmK, const PhaseAArgs a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ uint64_t bars[2];
    __shared__ uint32_t tmem_slot;
    __shared__ float s_scan[2];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int slot = blockIdx.x / a.n_heads, h = a.head_lo + blockIdx.x % a.n_heads;
    int seq, c;
    if (!slot_to_chunk(a.cu_seqlens, a.n_seq, slot, seq, c)) return;
    const int t_begin = a.cu_seqlens[seq], t_end = a.cu_seqlens[seq + 1];
    if (t_begin < 0 || t_end > a.total_T || t_end < t_begin) { if (tid == 0) atomicExch(a.status, 1); return; }
    const int t0 = t_begin + c * PA_CH;
    const int nrows = min(PA_CH, t_end - t0);

    const uint32_t sbase = smem_addr(smem);
    if (sbase & 1023u) { if (tid == 0) atomicExch(a.status, 4); return; }
    float* Lm = reinterpret_cast<float*>(smem + PA_SM_L);
    float* Tm = reinterpret_cast<float*>(smem + PA_SM_T);
    float* sLc = reinterpret_cast<float*>(smem + PA_SM_G);
    float* sBeta = sLc + 64;
    const uint32_t bar_k = smem_addr(&bars[0]), bar_mma = smem_addr(&bars[1]);

    if (tid == 0) {
        mbar_init(bar_k, 1); mbar_init(bar_mma, 1);
        fence_barrier_init();
        if (!FUSED) tma_prefetch_desc(&tmK);
    }
    if (warp == 0) { tmem_alloc(smem_addr(&tmem_slot), 64); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tb = tmem_slot;
    GDN_TSTAMP(0);

    float lgj = 0.f, bj = 0.f;                                       // log-decay and beta of token tid (threads 0..63)
    if (!FUSED) {
        if (tid == 0) {
            mbar_expect_tx(bar_k, 2 * 8192);
            tma_load_3d(sbase + PA_SM_K, &tmK, bar_k, 0, h, t0);
            tma_load_3d(sbase + PA_SM_K + 8192, &tmK, bar_k, 64, h, t0);
        }
        if (tid < nrows) { lgj = a.lg[(size_t)(t0 + tid) * a.H + h]; bj = a.beta[(size_t)(t0 + tid) * a.H + h]; }
    } else {
        // ---- conv (4 taps) + silu, q / k l2norm, gates: warp w owns tokens [16 w, 16 w + 16) of the tile; a lane owns 4 channels
        //      of each of q, k, v and slides a 4-row window of the raw mixed-qkv rows through registers ----
        const int tl0 = warp * 16;
        const float inv_scale = 0.08838834764831845f;
        const float e2 = 1e-6f * inv_scale * inv_scale;
        const float sc_q = bf(inv_scale * inv_scale), sc_k = bf(inv_scale);
        const int seq_t0 = t0 - t_begin;                            // position of the tile's first token inside its sequence
#pragma unroll 1
        for (int part = 0; part < 3 && tl0 < nrows; part++) {
            const int ch = part * KD + h * DK + lane * 4;
            float w[4][4];                                           // [channel][tap]
#pragma unroll
            for (int i = 0; i < 4; i++) unpack_bf16x4(*reinterpret_cast<const uint2*>(a.conv_w + (size_t)(ch + i) * 4), w[i]);
            auto raw_row = [&](int ts) -> uint2 {                    // raw row of sequence position ts (negative: the stored window)
                if (ts < 0) return *reinterpret_cast<const uint2*>(a.conv_state + ((size_t)seq * 3 + (ts + 3)) * CD + ch);
                return *reinterpret_cast<const uint2*>(a.proj + (size_t)(t_begin + ts) * a.row_stride + ch);
            };
            float x[4][4];                                           // [row in window][channel]
#pragma unroll
            for (int r = 0; r < 3; r++) unpack_bf16x4(raw_row(seq_t0 + tl0 - 3 + r), x[r]);
            __nv_bfloat16* dstbase = (part == 0 ? a.q : part == 1 ? a.k : a.v);
#pragma unroll 4
            for (int tt = 0; tt < 16; tt++) {
                const int tl = tl0 + tt;                             // token inside the tile
                if (tl >= nrows) break;
                unpack_bf16x4(raw_row(seq_t0 + tl), x[3]);
                float o[4], ss = 0.f;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    float acc = x[0][i] * w[i][0];
                    acc += x[1][i] * w[i][1];
                    acc += x[2][i] * w[i][2];
                    acc += x[3][i] * w[i][3];
                    o[i] = silu_bf16(bf(acc));
                    ss += o[i] * o[i];
                }
                if (part < 2) {
                    ss = warp_sum(ss);
                    const float rr = 1.0f / sqrtf(ss / (float)DK + e2);
                    const float sc = part == 0 ? sc_q : sc_k;
#pragma unroll
                    for (int i = 0; i < 4; i++) o[i] = bf(o[i] * rr) * sc;
                }
                uint2 pk;
                pk.x = pack_bf16x2(o[0], o[1]);
                pk.y = pack_bf16x2(o[2], o[3]);
                *reinterpret_cast<uint2*>(dstbase + ((size_t)(t0 + tl) * a.H + h) * DK + lane * 4) = pk;
                if (part == 1)                                       // k also goes to the operand tile: row tl, columns 4 lane .. 4 lane + 3
                    *reinterpret_cast<uint2*>(smem + PA_SM_K + (lane >> 4) * 8192 + sw128_offset(tl, (lane & 15) * 4)) = pk;
#pragma unroll
                for (int r = 0; r < 3; r++)
#pragma unroll
                    for (int i = 0; i < 4; i++) x[r][i] = x[r + 1][i];
            }
        }
        if (tid < nrows) {
            const __nv_bfloat16* prow = a.proj + (size_t)(t0 + tid) * a.row_stride;
            lgj = log_decay(expf(a.A_log[h]), ldbf(prow + CD + KD + HV + h), a.dt_bias[h]);
            bj = sigmoid_bf16(ldbf(prow + CD + KD + h));
        }
    }

    // ---- gates: Lc = inclusive prefix sum of the log2-decay over the 64 tokens (warps 0 and 1) ----
    float xs = lgj * 1.4426950408889634f;
    if (warp < 2) {
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const float y = __shfl_up_sync(0xffffffffu, xs, o); if (lane >= o) xs += y; }
        if (lane == 31) s_scan[warp] = xs;
    }
    // one warp polls the barrier (a poll loop costs issue slots that the five other resident blocks want); the block barrier below
    // hands the copy's writes on to the other warps
    if (!FUSED && warp == 0) {
        if (!pa_wait(bar_k, 0) && lane == 0) atomicExch(a.status, 3);
    }
    // rows past the end of the sequence are zero (qwen35/gdn_nax.py:55-60): a packed neighbour sequence must not leak in
    if (nrows < PA_CH) {
        const int nz = (PA_CH - nrows) * 8;
        for (int i = tid; i < 2 * nz; i += PA_THREADS) {
            const int tile = i / nz, p = i % nz;
            *reinterpret_cast<uint4*>(smem + PA_SM_K + tile * 8192 + nrows * 128 + p * 16) = make_uint4(0, 0, 0, 0);
        }
    }
    fence_proxy_async_smem();
    __syncthreads();
    if (warp == 1) xs += s_scan[0];
    GDN_TSTAMP(1);
    const float Ltot = s_scan[0] + s_scan[1];
    if (tid < 64) { sLc[tid] = xs; sBeta[tid] = bj; }

    // ---- G = K K^T on the tensor cores: M = 128 (rows 64..127 of the A operand read whatever follows the tile and are never used) ----
    if (tid == 0) {
        constexpr uint32_t I64 = idesc_bf16(128, 64, 0, 0);
#pragma unroll
        for (int ks = 0; ks < 8; ks++) {
            const uint64_t d = smem_desc_sw128(sbase + PA_SM_K + (ks >> 2) * 8192 + (ks & 3) * 32, 16, 1024);
            mma_ss(tb, d, d, I64, ks > 0);
        }
        mma_commit(bar_mma);
    }
    if (warp == 0) {
        if (!pa_wait(bar_mma, 0) && lane == 0) atomicExch(a.status, 3);      // (a product that never completed leaves garbage, not a fault)
    }
    __syncthreads();                                                 // Lc / beta and the finished product are visible to everyone
    tc_fence_after_sync();
    GDN_TSTAMP(2);

    // ---- raw K K^T rows out of tensor memory (threads 0..63 own TMEM lanes 0..63) ----
    if (tid < 64) {
#pragma unroll
        for (int half = 0; half < 2; half++) {
            uint32_t r[32];
            tmem_ld32(tb + ((uint32_t)(warp * 32) << 16) + half * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int jj = 0; jj < 32; jj += 4)
                *reinterpret_cast<float4*>(Lm + tid * PA_LS + half * 32 + jj) =
                    make_float4(__uint_as_float(r[jj]), __uint_as_float(r[jj + 1]), __uint_as_float(r[jj + 2]), __uint_as_float(r[jj + 3]));
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    GDN_TSTAMP(3);
    // ---- L[i][j] = beta_i 2^(Lc_i - Lc_j) G[i][j] for j < i, in place; thread = (row, half of the columns) ----
    {
        const int i = tid >> 1, hf = tid & 1;
        const float Li = sLc[i], bi = sBeta[i];
        float* row = Lm + i * PA_LS + hf * 32;
#pragma unroll
        for (int jj = 0; jj < 32; jj += 4) {
            const int j = hf * 32 + jj;
            float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
            if (j < i) {
                const float4 g = *reinterpret_cast<const float4*>(row + jj);
                const float4 lc = *reinterpret_cast<const float4*>(sLc + j);
                o.x = bi * pa_ex2(Li - lc.x) * g.x;
                o.y = (j + 1 < i) ? bi * pa_ex2(Li - lc.y) * g.y : 0.f;
                o.z = (j + 2 < i) ? bi * pa_ex2(Li - lc.z) * g.z : 0.f;
                o.w = (j + 3 < i) ? bi * pa_ex2(Li - lc.w) * g.w : 0.f;
            }
            *reinterpret_cast<float4*>(row + jj) = o;
        }
    }
    __syncthreads();

    // ---- T = (I + L)^-1 (T overwrites the K tile, which the tensor cores have finished reading) ----
    // (1) diagonal blocks: warp w inverts block w; lane j < 16 owns column j:  t_i = [i == j] - sum_{m < i} L[i][m] t_m.
    //     Lanes 16..31 of warps 0 and 2 zero the block to the right of theirs: steps (2) and (3) read whole 32 x 32 diagonal blocks.
    if (lane < 16) {
        const int b0 = warp * 16;
        // right-looking: once t_m is final, every later row takes its contribution -- sixteen independent accumulators, so the
        // dependent chain is one FMA per step instead of a whole row sum
        float t[16];
#pragma unroll
        for (int i = 0; i < 16; i++) t[i] = (i == lane) ? 1.f : 0.f;
        const float* lblk = Lm + b0 * PA_LS + b0;                     // broadcast reads: every lane needs the same L entries
#pragma unroll
        for (int m = 0; m < 15; m++) {
#pragma unroll
            for (int i = m + 1; i < 16; i++) t[i] -= lblk[i * PA_LS + m] * t[m];
        }
#pragma unroll
        for (int i = 0; i < 16; i++) Tm[(b0 + i) * PA_LS + b0 + lane] = t[i];
    } else if ((warp & 1) == 0) {
        const int b0 = warp * 16;
#pragma unroll
        for (int i = 0; i < 16; i++) Tm[(b0 + i) * PA_LS + b0 + lane] = 0.f;                      // columns b0 + 16 .. b0 + 31
    }
    __syncthreads();
    GDN_TSTAMP(4);
    // (2) blocks (1,0) and (3,2): T_ba = -T_bb (L_ba T_aa).  Warps 0, 1 take the first pair, warps 2, 3 the second; a warp owns 8 of
    //     the 16 columns.  The inner product replaces L_ba (nothing reads that block again).
    {
        const int pair = warp >> 1, n0 = (warp & 1) * 8;
        const int ra = pair * 32, rb = ra + 16;                       // first row of blocks a and b
        const int g = lane >> 2, t = lane & 3;
        float acc[1][4] = {{0.f, 0.f, 0.f, 0.f}};
        warp_mm_tf32x3<2, 1>(Lm + rb * PA_LS + ra, PA_LS, Tm + ra * PA_LS + ra + n0, PA_LS, lane, acc);
        __syncthreads();                                              // every warp has read its operand rows of L_ba
        *reinterpret_cast<float2*>(Lm + (rb + g) * PA_LS + ra + n0 + 2 * t) = make_float2(acc[0][0], acc[0][1]);
        *reinterpret_cast<float2*>(Lm + (rb + g + 8) * PA_LS + ra + n0 + 2 * t) = make_float2(acc[0][2], acc[0][3]);
        __syncthreads();
        float x[1][4] = {{0.f, 0.f, 0.f, 0.f}};
        warp_mm_tf32x3<2, 1>(Tm + rb * PA_LS + rb, PA_LS, Lm + rb * PA_LS + ra + n0, PA_LS, lane, x);      // T_bb has zeros above its diagonal
        *reinterpret_cast<float2*>(Tm + (rb + g) * PA_LS + ra + n0 + 2 * t) = make_float2(-x[0][0], -x[0][1]);
        *reinterpret_cast<float2*>(Tm + (rb + g + 8) * PA_LS + ra + n0 + 2 * t) = make_float2(-x[0][2], -x[0][3]);
    }
    __syncthreads();
    GDN_TSTAMP(5);
    // (3) the 32 x 32 block (rows 32..63, columns 0..31): T_ba = -T_hi (L_ba T_lo), T_lo / T_hi = the 32 x 32 diagonal blocks just
    //     completed; a warp owns a 16 x 16 quadrant of the result
    {
        const int r0 = (warp & 1) * 16, n0 = (warp >> 1) * 16;
        const int g = lane >> 2, t = lane & 3;
        float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        warp_mm_tf32x3<4, 2>(Lm + (32 + r0) * PA_LS, PA_LS, Tm + n0, PA_LS, lane, acc);
        __syncthreads();                                              // every warp has read its operand rows of L_ba
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
            *reinterpret_cast<float2*>(Lm + (32 + r0 + g) * PA_LS + n0 + 8 * nt + 2 * t) = make_float2(acc[nt][0], acc[nt][1]);
            *reinterpret_cast<float2*>(Lm + (32 + r0 + g + 8) * PA_LS + n0 + 8 * nt + 2 * t) = make_float2(acc[nt][2], acc[nt][3]);
        }
        __syncthreads();
        float x[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        warp_mm_tf32x3<4, 2>(Tm + (32 + r0) * PA_LS + 32, PA_LS, Lm + 32 * PA_LS + n0, PA_LS, lane, x);     // T_hi has zeros above its diagonal
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
            *reinterpret_cast<float2*>(Tm + (32 + r0 + g) * PA_LS + n0 + 8 * nt + 2 * t) = make_float2(-x[nt][0], -x[nt][1]);
            *reinterpret_cast<float2*>(Tm + (32 + r0 + g + 8) * PA_LS + n0 + 8 * nt + 2 * t) = make_float2(-x[nt][2], -x[nt][3]);
        }
    }
    __syncthreads();

    GDN_TSTAMP(6);
    // ---- record: Tb = T diag(beta) as bf16 hi / lo operand images, then the gate vectors ----
    unsigned char* rec = a.records + ((size_t)slot * a.H + h) * PA_REC_BYTES;
    {
        const int i = tid >> 1, hf = tid & 1;
#pragma unroll
        for (int cb = 0; cb < 4; cb++) {
            uint32_t bh[4] = {0u, 0u, 0u, 0u}, bl[4] = {0u, 0u, 0u, 0u};
            if (hf * 32 + cb * 8 <= i)                                // pieces entirely above the diagonal are zero: nothing to read or split
#pragma unroll
            for (int e = 0; e < 4; e += 2) {
                const int j = hf * 32 + cb * 8 + 2 * e;
                const float4 t4 = *reinterpret_cast<const float4*>(Tm + i * PA_LS + j);
                const float4 b4 = *reinterpret_cast<const float4*>(sBeta + j);
                // the lower triangle (diagonal included) is the result; everything above it is zero
                const float v0 = j <= i ? t4.x * b4.x : 0.f, v1 = j + 1 <= i ? t4.y * b4.y : 0.f;
                const float v2 = j + 2 <= i ? t4.z * b4.z : 0.f, v3 = j + 3 <= i ? t4.w * b4.w : 0.f;
                pa_split_pack(v0, v1, bh[e], bl[e]);
                pa_split_pack(v2, v3, bh[e + 1], bl[e + 1]);
            }
            const uint32_t o = i * 128 + (((hf * 4 + cb) ^ (i & 7)) << 4);
            *reinterpret_cast<uint4*>(rec + o) = make_uint4(bh[0], bh[1], bh[2], bh[3]);
            *reinterpret_cast<uint4*>(rec + 8192 + o) = make_uint4(bl[0], bl[1], bl[2], bl[3]);
        }
    }
    if (tid < 64) {
        float* gv = reinterpret_cast<float*>(rec + 16384);
        gv[tid] = xs;
        gv[64 + tid] = pa_ex2(xs);
        gv[128 + tid] = pa_ex2(Ltot - xs);
    }
    tc_fence_before_sync();
    __syncthreads();
    GDN_TSTAMP(7);
    if (warp == 0) tmem_dealloc(tb, 64);
}

// ----------------------------------------------------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------------------------------------------------
int make_token_map(CUtensorMap* m, const void* base, long long total_T, int H);      // gdn_prefill_sm100.cu

long long phase_a_slots(int n_seq, long long total_T) { return total_T / PA_CH + n_seq; }

size_t prefill_records_bytes(int n_seq, long long total_T, int H) {
    return (size_t)phase_a_slots(n_seq, total_T) * (size_t)H * PA_REC_BYTES;
}

int launch_phase_a(const void* k, const PhaseAArgs& a, bool fused, cudaStream_t stream) {
    if (a.n_seq <= 0 || a.n_heads <= 0) return GDN_OK;
    CUtensorMap tk;
    memset(&tk, 0, sizeof(tk));
    int rc;
    if (!fused && (rc = make_token_map(&tk, k, a.total_T, a.H))) return rc;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        if (cudaFuncSetAttribute(gdn_phase_a_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, PA_SM_TOTAL) != cudaSuccess ||
            cudaFuncSetAttribute(gdn_phase_a_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, PA_SM_TOTAL) != cudaSuccess)
            return check_launch("gdn_phase_a smem attribute");
        attr_set[dev] = true;
    }
    const long long blocks = phase_a_slots(a.n_seq, a.total_T) * a.n_heads;
    if (blocks > 0x7fffffffll) { set_error("gdn_phase_a: %lld tiles exceed the grid limit", blocks); return GDN_E_SHAPE; }
    if (fused) gdn_phase_a_kernel<true><<<(unsigned)blocks, PA_THREADS, PA_SM_TOTAL, stream>>>(tk, a);
    else       gdn_phase_a_kernel<false><<<(unsigned)blocks, PA_THREADS, PA_SM_TOTAL, stream>>>(tk, a);
    return check_launch("gdn_phase_a");
}

}  // namespace gdn

#ifdef GDN_TIMING
extern "C" __attribute__((visibility("default"))) int gdn_timing_log_a(long long* out_host, int n) {
    return cudaMemcpyFromSymbol(out_host, gdn::g_tlog, sizeof(long long) * n) == cudaSuccess ? 0 : -5;
}
#endif
