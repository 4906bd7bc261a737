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
// full-rate M = 128 MMA and a TMEM lane is one value row for the whole kernel:
//     G    [128 x 64]  = [K; Q] K^T            rows 0-63 = K K^T, rows 64-127 = Q K^T (K and Q tiles are stacked in smem)
//     P1^T [dv x 64]   = S0 K^T,  P2^T = S0 Q^T                         A = S0 (bf16 hi + lo) from TMEM
//     D^T  [dv x 64]   = V^T Tb^T + P1^T Tg^T,  Tg = -Tb diag(gamma)    A = V read MN-major from smem / P1^T (hi + lo) from TMEM
//     AD^T [dv x 64]   = D^T A^T                                        A = D^T (hi + lo) from TMEM, B = A (hi + lo) in smem
//     S    [dv x 128] += Dp^T K,  Dp = diag(dec) D                      A = Dp^T (hi + lo) in smem, B = K read MN-major
// The fp32 state lives in TMEM for the whole sequence.  Every operand that is derived from fp32 data (S, P1, D, Dp, Tb, Tg, A)
// is fed to the bf16 MMA as an exact hi + lo pair (16 significand bits), which keeps the final state within 1e-4 of fp64; K,
// Q and V are bf16 already.  (I + L)^-1 is an exact fp32 forward substitution (one column per thread), as in the reference
// (qwen35/gdn_nax.py:118-141); the tensor-core products with T are the "solve products".
//
// Roles (544 threads, one block per SM):
//   warps 0-3   "solver": everything that does not depend on the state, one chunk ahead of the chain: gates, L from K K^T,
//               the forward substitution, Tb / Tg
//   warps 4-11  "chain": the state-dependent passes between MMAs (two warps per TMEM lane quadrant, half of the columns each)
//   warp 12     lane 0 issues every tcgen05.mma
//   warps 13-16 "output": the A matrix from Q K^T, the y rows, and the TMA loads of the chunk after next
// The groups hand over through mbarriers (one arrival per warp); K/Q/V chunks arrive by TMA (128-byte swizzle, no multicast),
// double buffered; rows of a partial last chunk are zeroed in shared memory so that a packed neighbour sequence can never leak
// in.  Every wait is bounded: a wait that gives up sets the device status word and the block leaves.
#include <cuda.h>
// waiting warps sleep ~20 ns between polls of an mbarrier: back-to-back polls take issue slots and shared-memory bandwidth from
// the warps that do the work (measured: 5% of the kernel time)
#define GDN_POLL_SLEEP 20
#include "gdn_common.cuh"
#include "launchers.cuh"
#include "sm100_prims.cuh"

namespace gdn {

using namespace sm100;

constexpr int CH = 64;                               // chunk length
constexpr int PF_THREADS = 544;
// ---- shared memory map (bytes from a 1024-aligned base) ----
constexpr int SM_STAGE = 48 * 1024;                  // per stage: [K_h0 | Q_h0 | K_h1 | Q_h1] (4 x 8 KiB) + [V_h0 | V_h1] (2 x 8 KiB)
constexpr int SM_V = 32 * 1024;                      // offset of V inside a stage
constexpr int SM_TB_HI = 2 * SM_STAGE;               // Tb, Tg, A as bf16 hi / lo: [64][64], K-major, 8 KiB each
constexpr int SM_TB_LO = SM_TB_HI + 8192;
constexpr int SM_TG_HI = SM_TB_LO + 8192;
constexpr int SM_TG_LO = SM_TG_HI + 8192;
constexpr int SM_A_HI = SM_TG_LO + 8192;
constexpr int SM_A_LO = SM_A_HI + 8192;
constexpr int SM_DP_HI = SM_A_LO + 8192;             // Dp^T hi / lo: [128][64] bf16, K-major, 16 KiB each
constexpr int SM_DP_LO = SM_DP_HI + 16384;
constexpr int SM_L = SM_DP_LO + 16384;               // L fp32, column-major: Lt[j][i] = L[i][j], [64][LSTRIDE]
constexpr int LSTRIDE = 68;
constexpr int SM_T = SM_L + 64 * LSTRIDE * 4;        // T fp32 [64][LSTRIDE]
constexpr int SM_GATES = SM_T + 64 * LSTRIDE * 4;    // three sets (chunk mod 3) of Lc2, gamma, -gamma, dec, beta: [64] fp32 each
constexpr int GATE_SET = 5 * 64;                     // floats per set
constexpr int SM_TOTAL = SM_GATES + 3 * GATE_SET * 4 + 64;
// ---- tensor memory map (columns) ----
constexpr uint32_t TM_S = 0;                         // fp32 state, pre-scaled by the coming chunk's gamma_C   [128 cols]
constexpr uint32_t TM_SHI = 128, TM_SLO = 192;       // bf16 pairs of the unscaled state                        [64 + 64]
constexpr uint32_t TM_G = 256;                       // [K;Q] K^T                                               [64]
constexpr uint32_t TM_P1 = 320;                      // S0 K^T, later D^T                                       [64]
constexpr uint32_t TM_Y = 384;                       // S0 Q^T, scaled by gamma, then + A D = Y^T               [64]
constexpr uint32_t TM_ZHI = 448, TM_ZLO = 480;       // P1^T, later D^T, as bf16 pairs                          [32 + 32]
// ---- mbarriers ----
enum { B_KQV0 = 0, B_KQV1, B_INPUTS, B_GFREE, B_GDONE, B_TB, B_AREADY, B_YFREE, B_SREADY, B_P1DONE, B_ZREADY, B_DDONE, B_DPREADY, B_SDONE,
       B_YSCALED, B_YDONE, B_AGRP, B_COUNT };

constexpr float LOG2E = 1.4426950408889634f;
constexpr uint32_t WAIT_LIMIT = 200000u;               // polls of up to ~20 us each

__device__ __forceinline__ float ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }

__device__ __forceinline__ void split_pack(float x0, float x1, uint32_t& hi, uint32_t& lo) {
    hi = pack_bf16x2(x0, x1);
    lo = pack_bf16x2(x0 - __uint_as_float(hi << 16), x1 - __uint_as_float(hi & 0xffff0000u));
}

// Exact forward substitution for column j of T = (I + L)^-1 (x_i = [i == j] - sum_{m < i} L[i][m] x_m), 16 rows at a time, two
// threads per column.  The contribution of all earlier rows is a rolled loop that the two threads of a column split by the
// parity of m (x_m is read back from the column's own entries of Tm; L comes as the column-major copy Lt[m][i], so 16 rows of
// one column are four broadcast float4 loads); the 16 x 16 triangle inside the block is unrolled and done by both threads.
// Sixteen independent accumulators keep the FMA pipe busy.  The block loop is deliberately NOT unrolled and nothing is
// specialised per warp: the whole routine is ~400 instructions that every block and every warp re-executes, whereas a fully
// unrolled 64 x 64 substitution (or one copy per warp) streams tens of KiB of straight-line code through the instruction cache
// for every chunk and runs several times slower.  b0 = first 16-row block that can be non-zero for the columns of this warp.
__device__ __forceinline__ void solve_column(const float* __restrict__ Lt, float* __restrict__ Tm, int j, int p, int b0) {
    if (p == 0)
        for (int i = 0; i < 16 * b0; i++) Tm[i * LSTRIDE + j] = 0.f;
#pragma unroll 1
    for (int b = b0; b < 4; b++) {
        float acc[16];
#pragma unroll
        for (int ii = 0; ii < 16; ii++) acc[ii] = (p == 0 && 16 * b + ii == j) ? 1.f : 0.f;
        if (b > b0) {
#pragma unroll 4
            for (int m = 16 * b0 + p; m < 16 * b; m += 2) {
                const float xm = Tm[m * LSTRIDE + j];
                const float4* lp = reinterpret_cast<const float4*>(Lt + m * LSTRIDE + 16 * b);
#pragma unroll
                for (int v4 = 0; v4 < 4; v4++) {
                    const float4 l = lp[v4];
                    acc[4 * v4] -= l.x * xm; acc[4 * v4 + 1] -= l.y * xm; acc[4 * v4 + 2] -= l.z * xm; acc[4 * v4 + 3] -= l.w * xm;
                }
            }
#pragma unroll
            for (int ii = 0; ii < 16; ii++) acc[ii] += __shfl_xor_sync(0xffffffffu, acc[ii], 1);
        }
        const float* lblk = Lt + (16 * b) * LSTRIDE + 16 * b;        // Lt[16b + ii][16b + kk] = L[16b + kk][16b + ii]
        float* tcol = Tm + (16 * b) * LSTRIDE + j;
        // right-looking elimination inside the block; the column of step ii + 1 is fetched before the FMAs of step ii, so the
        // loop-carried dependence is a single FMA per step (no store inside the loop: stores would pin the loads in place)
        float4 cur[4], nxt[4];
#pragma unroll
        for (int v4 = 0; v4 < 4; v4++) cur[v4] = *reinterpret_cast<const float4*>(lblk + 4 * v4);
#pragma unroll
        for (int ii = 0; ii < 16; ii++) {
            if (ii + 1 < 16) {
#pragma unroll
                for (int v4 = (ii + 2) / 4; v4 < 4; v4++) nxt[v4] = *reinterpret_cast<const float4*>(lblk + (ii + 1) * LSTRIDE + 4 * v4);
            }
            const float x = acc[ii];
#pragma unroll
            for (int v4 = (ii + 1) / 4; v4 < 4; v4++) {
                const float4 l = cur[v4];
                if (4 * v4 > ii) acc[4 * v4] -= l.x * x;
                if (4 * v4 + 1 > ii) acc[4 * v4 + 1] -= l.y * x;
                if (4 * v4 + 2 > ii) acc[4 * v4 + 2] -= l.z * x;
                if (4 * v4 + 3 > ii) acc[4 * v4 + 3] -= l.w * x;
            }
#pragma unroll
            for (int v4 = 0; v4 < 4; v4++) cur[v4] = nxt[v4];
        }
        if (p == 0) {
#pragma unroll
            for (int ii = 0; ii < 16; ii++) tcol[ii * LSTRIDE] = acc[ii];
        }
        __syncwarp();
    }
}

__global__ void __launch_bounds__(PF_THREADS, 1)
gdn_prefill_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                   const PrefillArgs a) {
    // the swizzled tiles need a 1024-byte aligned base; the declared alignment provides it (checked below).  The array is used
    // directly, not through a re-aligned pointer, so that the compiler keeps every access in the shared address space
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ uint64_t bars[B_COUNT];
    __shared__ uint32_t tmem_slot;
    __shared__ float s_scan[4];
    __shared__ int s_abort;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int seq = blockIdx.x / a.n_heads, h = a.head_lo + blockIdx.x % a.n_heads;
    const int t_begin = a.cu_seqlens[seq], t_end = a.cu_seqlens[seq + 1];
    const int len = t_end - t_begin;
    const float* init_head = nullptr;
    if (a.init_state) {
        const int ii = a.init_idx ? a.init_idx[seq] : seq;
        if (ii >= 0) init_head = a.init_state + ((size_t)ii * a.H + h) * DV * DK;
    }
    float* fin_head = a.final_state + ((size_t)seq * a.H + h) * DV * DK;
    if (len <= 0 || t_begin < 0 || t_end > a.total_T) {
        if (len < 0 || t_begin < 0 || t_end > a.total_T) { if (tid == 0) atomicExch(a.status, 1); return; }
        for (int i = tid * 4; i < DV * DK; i += PF_THREADS * 4)       // nothing to compute: the state passes through unchanged
            *reinterpret_cast<float4*>(fin_head + i) = init_head ? *reinterpret_cast<const float4*>(init_head + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        return;
    }
    const int nchunks = (len + CH - 1) / CH;

    const uint32_t sbase = smem_addr(smem);
    if (sbase & 1023u) { if (tid == 0) atomicExch(a.status, 4); return; }
    auto bar = [&](int i) -> uint32_t { return smem_addr(&bars[i]); };
    float* Lm = reinterpret_cast<float*>(smem + SM_L);
    float* Tm = reinterpret_cast<float*>(smem + SM_T);
    float* gates_base = reinterpret_cast<float*>(smem + SM_GATES);
    // gate arrays of chunk c: Lc2 (cumulative log2-decay), gamma, -gamma, dec, beta.  Three sets: the solver writes set c while
    // the chain may still read set c-1 and c-2 is certainly retired (the solver has seen the D MMAs of chunk c-2 complete, and
    // those were issued after every reader of set c-3 had finished)
    auto g_Lc = [&](int c) -> float* { return gates_base + (c % 3) * GATE_SET; };
    auto g_gam = [&](int c) -> float* { return gates_base + (c % 3) * GATE_SET + 64; };
    auto g_ngam = [&](int c) -> float* { return gates_base + (c % 3) * GATE_SET + 128; };
    auto g_dec = [&](int c) -> float* { return gates_base + (c % 3) * GATE_SET + 192; };
    auto g_beta = [&](int c) -> float* { return gates_base + (c % 3) * GATE_SET + 256; };

    if (tid == 0) {
        mbar_init(bar(B_KQV0), 1); mbar_init(bar(B_KQV1), 1);
        mbar_init(bar(B_INPUTS), 4); mbar_init(bar(B_TB), 4); mbar_init(bar(B_AGRP), 4);
        mbar_init(bar(B_GFREE), 4); mbar_init(bar(B_AREADY), 2); mbar_init(bar(B_YFREE), 4);
        mbar_init(bar(B_SREADY), 8); mbar_init(bar(B_ZREADY), 8); mbar_init(bar(B_DPREADY), 8); mbar_init(bar(B_YSCALED), 8);
        mbar_init(bar(B_GDONE), 1); mbar_init(bar(B_P1DONE), 1); mbar_init(bar(B_DDONE), 1); mbar_init(bar(B_SDONE), 1); mbar_init(bar(B_YDONE), 1);
        s_abort = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
    }
    if (warp == 0) { tmem_alloc(smem_addr(&tmem_slot), 512); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tb = tmem_slot;

    auto issue_tma = [&](int c) {                                    // one thread: K, Q, V of chunk c -> stage c & 1
        const uint32_t st = sbase + (c & 1) * SM_STAGE;
        const uint32_t kb = bar((c & 1) ? B_KQV1 : B_KQV0);
        const int t0 = t_begin + c * CH;
        mbar_expect_tx(kb, 6 * 8192);
        tma_load_3d(st, &tmK, kb, 0, h, t0);
        tma_load_3d(st + 8192, &tmQ, kb, 0, h, t0);
        tma_load_3d(st + 16384, &tmK, kb, 64, h, t0);
        tma_load_3d(st + 24576, &tmQ, kb, 64, h, t0);
        tma_load_3d(st + SM_V, &tmV, kb, 0, h, t0);
        tma_load_3d(st + SM_V + 8192, &tmV, kb, 64, h, t0);
    };
    // one arrival per warp: every lane has already fenced its own writes, the warp barrier orders them before lane 0's arrive
    auto warp_arrive = [&](int b) {
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(b));
    };
    // a bounded wait; on failure the whole block is told to leave
    auto wait = [&](int b, uint32_t parity) -> bool {
        if (mbar_wait(bar(b), parity & 1u, WAIT_LIMIT)) return true;
        atomicExch(&s_abort, 1);
        atomicExch(a.status, 3);
        return false;
    };
    auto aborted = [&]() -> bool { return *(volatile int*)&s_abort != 0; };

    if (warp < 4) {
        // ============================================================================================================
        // solver: gates, L, T = (I + L)^-1, Tb / Tg -- runs up to one chunk ahead of the chain
        // ============================================================================================================
        const uint32_t tl = tb + ((uint32_t)(warp * 32) << 16);
        uint32_t grp_phase = 0;
        auto group_sync = [&]() -> bool {                            // barrier among the 4 warps, bounded like every other wait
            warp_arrive(B_AGRP);
            const bool okw = wait(B_AGRP, grp_phase);
            grp_phase ^= 1u;
            return okw;
        };
        // gate inputs are fetched one chunk ahead so that their latency hides behind the previous chunk's work
        float lg_pre = 0.f, b_pre = 0.f;
        if (tid < 64 && t_begin + tid < t_end) { lg_pre = a.lg[(size_t)(t_begin + tid) * a.H + h]; b_pre = a.beta[(size_t)(t_begin + tid) * a.H + h]; }
        for (int c = 0; c < nchunks; c++) {
            const int stage = c & 1;
            const int t0 = t_begin + c * CH;
            const int nrows = min(CH, t_end - t0);
            if (aborted()) break;
            // ---- gates: Lc2 = inclusive prefix sum of the log2-decay, gamma, dec, beta ----
            const float lgj = lg_pre * LOG2E, bj = b_pre;
            lg_pre = 0.f; b_pre = 0.f;
            if (tid < 64 && t0 + CH + tid < t_end) { lg_pre = a.lg[(size_t)(t0 + CH + tid) * a.H + h]; b_pre = a.beta[(size_t)(t0 + CH + tid) * a.H + h]; }
            float xs = lgj;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const float y = __shfl_up_sync(0xffffffffu, xs, o); if (lane >= o) xs += y; }
            if (lane == 31 && warp < 2) s_scan[warp] = xs;
            if (!group_sync()) break;
            if (warp == 1) xs += s_scan[0];
            const float Ltot = s_scan[0] + s_scan[1];
            if (tid < 64) {
                const float g = ex2(xs);
                g_Lc(c)[tid] = xs; g_gam(c)[tid] = g; g_ngam(c)[tid] = -g; g_dec(c)[tid] = ex2(Ltot - xs); g_beta(c)[tid] = bj;
            }
            if (!wait(stage ? B_KQV1 : B_KQV0, (uint32_t)(c >> 1))) break;
            if (nrows < CH) {
                // rows past the end of the sequence are zero (qwen35/gdn_nax.py:55-60): 6 tiles x (64 - nrows) rows x 128 B
                const int nz = (CH - nrows) * 8;
                for (int i = tid; i < 6 * nz; i += 128) {
                    const int tile = i / nz, p = i % nz;
                    *reinterpret_cast<uint4*>(smem + stage * SM_STAGE + tile * 8192 + nrows * 128 + p * 16) = make_uint4(0, 0, 0, 0);
                }
                fence_proxy_async_smem();
            }
            tc_fence_before_sync();                                  // this group's reads of the previous G are complete
            warp_arrive(B_INPUTS);

            // ---- L from G = [K;Q] K^T (lanes 0..63), stored column-major in fp32 ----
            if (!wait(B_GDONE, (uint32_t)c)) break;
            tc_fence_after_sync();
            if (!group_sync()) break;                                // gates are visible to the whole group
            if (tid < 64) {
                const int i = tid;
                const float* Lc = g_Lc(c);
                const float Li = Lc[i], bi = g_beta(c)[i];
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    uint32_t r[32];
                    tmem_ld32(tl + TM_G + half * 32, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int jj = 0; jj < 32; jj += 4) {
                        const float4 lc = *reinterpret_cast<const float4*>(Lc + half * 32 + jj);
                        const int j = half * 32 + jj;
                        Lm[j * LSTRIDE + i] = (j < i) ? bi * ex2(Li - lc.x) * __uint_as_float(r[jj]) : 0.f;
                        Lm[(j + 1) * LSTRIDE + i] = (j + 1 < i) ? bi * ex2(Li - lc.y) * __uint_as_float(r[jj + 1]) : 0.f;
                        Lm[(j + 2) * LSTRIDE + i] = (j + 2 < i) ? bi * ex2(Li - lc.z) * __uint_as_float(r[jj + 2]) : 0.f;
                        Lm[(j + 3) * LSTRIDE + i] = (j + 3 < i) ? bi * ex2(Li - lc.w) * __uint_as_float(r[jj + 3]) : 0.f;
                    }
                }
            }
            tc_fence_before_sync();
            if (!group_sync()) break;

            // ---- T = (I + L)^-1: two threads per column ----
            solve_column(Lm, Tm, tid >> 1, tid & 1, warp);
            if (!group_sync()) break;
            // ---- Tb = T diag(beta), Tg = -Tb diag(gamma) as bf16 hi/lo K-major rows: thread = (row, half of the columns) ----
            if (c >= 1 && !wait(B_DDONE, (uint32_t)(c - 1))) break;  // the previous chunk's D MMAs have read the old Tb / Tg
            {
                const int i = tid >> 1, hf = tid & 1;
                const float* be = g_beta(c);
                const float* ng = g_ngam(c);
#pragma unroll
                for (int cb = 0; cb < 4; cb++) {
                    uint32_t bh[4], bl[4], gh[4], gl[4];
#pragma unroll
                    for (int e = 0; e < 4; e += 2) {
                        const int j = hf * 32 + cb * 8 + 2 * e;
                        const float4 t4 = *reinterpret_cast<const float4*>(Tm + i * LSTRIDE + j);
                        const float4 b4 = *reinterpret_cast<const float4*>(be + j);
                        const float4 g4 = *reinterpret_cast<const float4*>(ng + j);
                        const float v0 = t4.x * b4.x, v1 = t4.y * b4.y, v2 = t4.z * b4.z, v3 = t4.w * b4.w;
                        split_pack(v0, v1, bh[e], bl[e]);
                        split_pack(v2, v3, bh[e + 1], bl[e + 1]);
                        split_pack(v0 * g4.x, v1 * g4.y, gh[e], gl[e]);
                        split_pack(v2 * g4.z, v3 * g4.w, gh[e + 1], gl[e + 1]);
                    }
                    const uint32_t o = i * 128 + (((hf * 4 + cb) ^ (i & 7)) << 4);
                    *reinterpret_cast<uint4*>(smem + SM_TB_HI + o) = make_uint4(bh[0], bh[1], bh[2], bh[3]);
                    *reinterpret_cast<uint4*>(smem + SM_TB_LO + o) = make_uint4(bl[0], bl[1], bl[2], bl[3]);
                    *reinterpret_cast<uint4*>(smem + SM_TG_HI + o) = make_uint4(gh[0], gh[1], gh[2], gh[3]);
                    *reinterpret_cast<uint4*>(smem + SM_TG_LO + o) = make_uint4(gl[0], gl[1], gl[2], gl[3]);
                }
            }
            fence_proxy_async_smem();
            warp_arrive(B_TB);
        }
    } else if (warp < 12) {
        // ============================================================================================================
        // chain: the state-dependent passes between the MMAs: two warps per TMEM lane quadrant, half of the columns each
        // ============================================================================================================
        const int cw = warp - 4, q = cw & 3, hf = cw >> 2;
        const int r = q * 32 + lane;                                 // value row of this thread
        const uint32_t tl = tb + ((uint32_t)(q * 32) << 16);
        // this lane's share of the log-decay of chunk c (two rows); summed over the warp it is the chunk's total.  The loads are
        // issued one chunk before the value is needed.
        auto decay_part = [&](int c) -> float {
            float x = 0.f;
            const int t = t_begin + c * CH + lane;
            if (c < nchunks) {
                if (t < t_end) x = a.lg[(size_t)t * a.H + h];
                if (t + 32 < t_end) x += a.lg[(size_t)(t + 32) * a.H + h];
            }
            return x;
        };
        float part_next = decay_part(1);
        // ---- initial state -> TMEM: unscaled bf16 hi/lo pairs and the fp32 copy pre-scaled by gamma_C of chunk 0 ----
        {
            const float gC0 = ex2(warp_sum(decay_part(0)) * LOG2E);
            const float* init = init_head ? init_head + (size_t)r * DK + hf * 64 : nullptr;
#pragma unroll
            for (int blk = 0; blk < 2; blk++) {
                uint32_t rr[32], hi[16], lo[16];
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    const float4 v4 = init ? *reinterpret_cast<const float4*>(init + blk * 32 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                    split_pack(v4.x, v4.y, hi[i / 2], lo[i / 2]);
                    split_pack(v4.z, v4.w, hi[i / 2 + 1], lo[i / 2 + 1]);
                    rr[i] = __float_as_uint(v4.x * gC0); rr[i + 1] = __float_as_uint(v4.y * gC0);
                    rr[i + 2] = __float_as_uint(v4.z * gC0); rr[i + 3] = __float_as_uint(v4.w * gC0);
                }
                tmem_st32(tl + TM_S + hf * 64 + blk * 32, rr);
                tmem_st16(tl + TM_SHI + hf * 32 + blk * 16, hi);
                tmem_st16(tl + TM_SLO + hf * 32 + blk * 16, lo);
            }
            tmem_wait_st();
            tc_fence_before_sync();
            warp_arrive(B_SREADY);
        }
        for (int c = 0; c < nchunks; c++) {
            const uint32_t par = (uint32_t)c;
            const bool last = c == nchunks - 1;
            if (aborted()) break;
            const float gC_next = last ? 1.f : ex2(warp_sum(part_next) * LOG2E);
            part_next = decay_part(c + 2);

            // ---- P1^T -> bf16 hi/lo pairs in TMEM (the A operand of P1^T Tg^T) ----
            if (!wait(B_P1DONE, par)) break;
            tc_fence_after_sync();
            {
                uint32_t rr[32], hi[16], lo[16];
                tmem_ld32(tl + TM_P1 + hf * 32, rr);
                tmem_wait_ld();
#pragma unroll
                for (int jj = 0; jj < 32; jj += 2) split_pack(__uint_as_float(rr[jj]), __uint_as_float(rr[jj + 1]), hi[jj / 2], lo[jj / 2]);
                tmem_st16(tl + TM_ZHI + hf * 16, hi);
                tmem_st16(tl + TM_ZLO + hf * 16, lo);
                tmem_wait_st();
            }
            tc_fence_before_sync();
            warp_arrive(B_ZREADY);

            // ---- D^T -> bf16 hi/lo pairs in TMEM (A operand of A D) and Dp^T = D^T diag(dec) -> hi/lo K-major rows in smem ----
            if (!wait(B_DDONE, par)) break;
            tc_fence_after_sync();
            {
                const float* dec = g_dec(c);
                uint32_t rr[32], hi[16], lo[16];
                tmem_ld32(tl + TM_P1 + hf * 32, rr);
                tmem_wait_ld();
#pragma unroll
                for (int jj = 0; jj < 32; jj += 2) split_pack(__uint_as_float(rr[jj]), __uint_as_float(rr[jj + 1]), hi[jj / 2], lo[jj / 2]);
                tmem_st16(tl + TM_ZHI + hf * 16, hi);
                tmem_st16(tl + TM_ZLO + hf * 16, lo);
#pragma unroll
                for (int cb = 0; cb < 4; cb++) {
                    uint32_t ph[4], pl[4];
#pragma unroll
                    for (int e = 0; e < 4; e += 2) {
                        const int jj = cb * 8 + 2 * e;
                        const float4 d4 = *reinterpret_cast<const float4*>(dec + hf * 32 + jj);
                        split_pack(__uint_as_float(rr[jj]) * d4.x, __uint_as_float(rr[jj + 1]) * d4.y, ph[e], pl[e]);
                        split_pack(__uint_as_float(rr[jj + 2]) * d4.z, __uint_as_float(rr[jj + 3]) * d4.w, ph[e + 1], pl[e + 1]);
                    }
                    const uint32_t o = r * 128 + (((hf * 4 + cb) ^ (r & 7)) << 4);
                    *reinterpret_cast<uint4*>(smem + SM_DP_HI + o) = make_uint4(ph[0], ph[1], ph[2], ph[3]);
                    *reinterpret_cast<uint4*>(smem + SM_DP_LO + o) = make_uint4(pl[0], pl[1], pl[2], pl[3]);
                }
                tmem_wait_st();
            }
            fence_proxy_async_smem();
            tc_fence_before_sync();
            warp_arrive(B_DPREADY);

            // ---- after the state update: scale P2^T by gamma (A D is accumulated on top of it), then the new state ----
            if (!wait(B_SDONE, par)) break;
            tc_fence_after_sync();
            {
                const float* gam = g_gam(c);
                uint32_t rr[32];
                tmem_ld32(tl + TM_Y + hf * 32, rr);
                tmem_wait_ld();
#pragma unroll
                for (int ii = 0; ii < 32; ii += 4) {
                    const float4 g4 = *reinterpret_cast<const float4*>(gam + hf * 32 + ii);
                    rr[ii] = __float_as_uint(__uint_as_float(rr[ii]) * g4.x); rr[ii + 1] = __float_as_uint(__uint_as_float(rr[ii + 1]) * g4.y);
                    rr[ii + 2] = __float_as_uint(__uint_as_float(rr[ii + 2]) * g4.z); rr[ii + 3] = __float_as_uint(__uint_as_float(rr[ii + 3]) * g4.w);
                }
                tmem_st32(tl + TM_Y + hf * 32, rr);
                tmem_wait_st();
            }
            tc_fence_before_sync();
            warp_arrive(B_YSCALED);
            // bf16 hi/lo pairs of the new state for the next chunk's products, fp32 copy pre-scaled by the next gamma_C (or the output)
#pragma unroll
            for (int blk = 0; blk < 2; blk++) {
                uint32_t rr[32], hi[16], lo[16];
                tmem_ld32(tl + TM_S + hf * 64 + blk * 32, rr);
                tmem_wait_ld();
                if (last) {
                    float* fin = fin_head + (size_t)r * DK + hf * 64 + blk * 32;
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *reinterpret_cast<float4*>(fin + i) = make_float4(__uint_as_float(rr[i]), __uint_as_float(rr[i + 1]), __uint_as_float(rr[i + 2]),
                                                                         __uint_as_float(rr[i + 3]));
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) split_pack(__uint_as_float(rr[i]), __uint_as_float(rr[i + 1]), hi[i / 2], lo[i / 2]);
#pragma unroll
                    for (int i = 0; i < 32; i++) rr[i] = __float_as_uint(__uint_as_float(rr[i]) * gC_next);
                    tmem_st16(tl + TM_SHI + hf * 32 + blk * 16, hi);
                    tmem_st16(tl + TM_SLO + hf * 32 + blk * 16, lo);
                    tmem_st32(tl + TM_S + hf * 64 + blk * 32, rr);
                }
            }
            if (!last) {
                tmem_wait_st();
                tc_fence_before_sync();
                warp_arrive(B_SREADY);
            }
        }
    } else if (warp == 12) {
        // ============================================================================================================
        // the MMA issuer (one thread)
        // ============================================================================================================
        if (lane == 0) {
            constexpr uint32_t I64 = idesc_bf16(128, 64, 0, 0);      // N = 64, A and B K-major (A may also come from TMEM)
            constexpr uint32_t I64_AMN = idesc_bf16(128, 64, 1, 0);  // N = 64, A read MN-major (V as V^T)
            constexpr uint32_t I128_BMN = idesc_bf16(128, 128, 0, 1);// N = 128, B read MN-major (K as the [tokens x dk] factor)
            auto issue_G = [&](int c) {                              // G = [K; Q] K^T of chunk c
                const uint32_t st = sbase + (c & 1) * SM_STAGE;
#pragma unroll
                for (int ks = 0; ks < 8; ks++) {
                    const uint32_t off = (ks >> 2) * 16384 + (ks & 3) * 32;
                    const uint64_t d = smem_desc_sw128(st + off, 16, 1024);
                    mma_ss(tb + TM_G, d, d, I64, ks > 0);
                }
                mma_commit(bar(B_GDONE));
            };
            issue_tma(0);
            if (nchunks > 1) issue_tma(1);
            bool ok = wait(B_INPUTS, 0);
            if (ok) { tc_fence_after_sync(); issue_G(0); }
            for (int c = 0; ok && c < nchunks; c++) {
                const uint32_t par = (uint32_t)c;
                const uint32_t st = sbase + (c & 1) * SM_STAGE;
                if (aborted()) break;
                // ---- P1^T = S0 K^T (S0 = hi + lo from TMEM) ----
                if (!wait(B_SREADY, par)) break;
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
                mma_commit(bar(B_P1DONE));
                // ---- G of the next chunk, so that the solver works one chunk ahead ----
                if (c + 1 < nchunks) {
                    if (!wait(B_INPUTS, par + 1) || !wait(B_GFREE, par)) break;
                    tc_fence_after_sync();
                    issue_G(c + 1);
                }
                // ---- D^T = V^T Tb^T + P1^T Tg^T (the P1 columns become the D accumulator once P1 has been split) ----
                if (!wait(B_TB, par) || !wait(B_ZREADY, par)) break;
                tc_fence_after_sync();
#pragma unroll
                for (int part = 0; part < 2; part++) {
                    const uint32_t bsm = sbase + (part ? SM_TB_LO : SM_TB_HI);
#pragma unroll
                    for (int ks = 0; ks < 4; ks++)
                        mma_ss(tb + TM_P1, smem_desc_sw128(st + SM_V + ks * 2048, 8192, 1024), smem_desc_sw128(bsm + ks * 32, 16, 1024), I64_AMN,
                               (part | ks) != 0);
                }
#pragma unroll
                for (int term = 0; term < 3; term++) {
                    const uint32_t acol = term == 1 ? TM_ZLO : TM_ZHI;
                    const uint32_t bsm = sbase + (term == 2 ? SM_TG_LO : SM_TG_HI);
#pragma unroll
                    for (int ks = 0; ks < 4; ks++) mma_ts(tb + TM_P1, tb + acol + ks * 8, smem_desc_sw128(bsm + ks * 32, 16, 1024), I64, 1);
                }
                mma_commit(bar(B_DDONE));
                // ---- P2^T = S0 Q^T (once the previous y has left its columns), then the state update S += Dp^T K ----
                if (!wait(B_DPREADY, par)) break;
                if (c >= 1 && !wait(B_YFREE, par - 1)) break;
                tc_fence_after_sync();
#pragma unroll
                for (int part = 0; part < 2; part++) {
                    const uint32_t acol = part ? TM_SLO : TM_SHI;
#pragma unroll
                    for (int ks = 0; ks < 8; ks++) {
                        const uint32_t off = 8192 + (ks >> 2) * 16384 + (ks & 3) * 32;
                        mma_ts(tb + TM_Y, tb + acol + ks * 8, smem_desc_sw128(st + off, 16, 1024), I64, (part | ks) != 0);
                    }
                }
#pragma unroll
                for (int part = 0; part < 2; part++) {
                    const uint32_t asm_ = sbase + (part ? SM_DP_LO : SM_DP_HI);
#pragma unroll
                    for (int ks = 0; ks < 4; ks++)
                        mma_ss(tb + TM_S, smem_desc_sw128(asm_ + ks * 32, 16, 1024), smem_desc_sw128(st + ks * 2048, 16384, 1024), I128_BMN, 1);
                }
                mma_commit(bar(B_SDONE));
                // ---- Y^T = gamma-scaled P2^T + D^T A^T ----
                if (!wait(B_AREADY, par) || !wait(B_YSCALED, par)) break;
                tc_fence_after_sync();
#pragma unroll
                for (int term = 0; term < 3; term++) {
                    const uint32_t acol = term == 1 ? TM_ZLO : TM_ZHI;
                    const uint32_t bsm = sbase + (term == 2 ? SM_A_LO : SM_A_HI);
#pragma unroll
                    for (int ks = 0; ks < 4; ks++) mma_ts(tb + TM_Y, tb + acol + ks * 8, smem_desc_sw128(bsm + ks * 32, 16, 1024), I64, 1);
                }
                mma_commit(bar(B_YDONE));
            }
        }
    } else {
        // ============================================================================================================
        // output: A from Q K^T (the two warps that own TMEM lanes 64..127), y rows, TMA of the chunk after next
        // ============================================================================================================
        const int q = warp & 3;
        const int r = q * 32 + lane;
        const uint32_t tl = tb + ((uint32_t)(q * 32) << 16);
        for (int c = 0; c < nchunks; c++) {
            const uint32_t par = (uint32_t)c;
            const int t0 = t_begin + c * CH;
            const int nrows = min(CH, t_end - t0);
            if (aborted()) break;
            // ---- A = lower_incl(exp(Lc_i - Lc_j) Q K^T) as bf16 hi/lo K-major rows (the previous chunk's A D has completed) ----
            if (!wait(B_GDONE, par)) break;
            tc_fence_after_sync();
            if (q >= 2) {
                const int i = r - 64;
                const float* Lc = g_Lc(c);
                const float Li = Lc[i];
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    uint32_t rr[32];
                    tmem_ld32(tl + TM_G + half * 32, rr);
                    tmem_wait_ld();
#pragma unroll
                    for (int cb = 0; cb < 4; cb++) {                  // 16-byte pieces: 8 columns each
                        uint32_t hi[4], lo[4];
#pragma unroll
                        for (int e = 0; e < 4; e += 2) {
                            const int jj = cb * 8 + 2 * e, j = half * 32 + jj;
                            const float4 lc = *reinterpret_cast<const float4*>(Lc + j);
                            const float a0 = (j <= i) ? ex2(Li - lc.x) * __uint_as_float(rr[jj]) : 0.f;
                            const float a1 = (j + 1 <= i) ? ex2(Li - lc.y) * __uint_as_float(rr[jj + 1]) : 0.f;
                            const float a2 = (j + 2 <= i) ? ex2(Li - lc.z) * __uint_as_float(rr[jj + 2]) : 0.f;
                            const float a3 = (j + 3 <= i) ? ex2(Li - lc.w) * __uint_as_float(rr[jj + 3]) : 0.f;
                            split_pack(a0, a1, hi[e], lo[e]);
                            split_pack(a2, a3, hi[e + 1], lo[e + 1]);
                        }
                        const uint32_t o = i * 128 + (((half * 4 + cb) ^ (i & 7)) << 4);
                        *reinterpret_cast<uint4*>(smem + SM_A_HI + o) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                        *reinterpret_cast<uint4*>(smem + SM_A_LO + o) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                    }
                }
                fence_proxy_async_smem();
                tc_fence_before_sync();
                warp_arrive(B_AREADY);
                warp_arrive(B_GFREE);
            } else {
                // every warp that waits on B_GDONE must have seen phase c before phase c + 1 may complete: a warp that falls a
                // whole phase behind would mistake phase c + 2 for phase c (the parity repeats) and the block would stall
                warp_arrive(B_GFREE);
            }
            // ---- y[t0 + i, h, v] = Y^T[v][i]: each lane owns one value row, a warp store covers 64 contiguous bytes ----
            if (!wait(B_YDONE, par)) break;
            tc_fence_after_sync();
            if (warp == 13 && lane == 0 && c + 2 < nchunks) issue_tma(c + 2);    // every reader of this stage (MMAs of chunk c) has finished
            {
                __nv_bfloat16* yp = a.y + ((size_t)t0 * a.H + h) * DV + r;
                uint32_t y0[32], y1[32];
                tmem_ld32(tl + TM_Y, y0);
                tmem_ld32(tl + TM_Y + 32, y1);
                tmem_wait_ld();
                tc_fence_before_sync();
                warp_arrive(B_YFREE);                                // the columns may take the next chunk's P2
#pragma unroll
                for (int ii = 0; ii < 32; ii++)
                    if (ii < nrows) yp[(size_t)ii * a.H * DV] = __float2bfloat16_rn(__uint_as_float(y0[ii]));
#pragma unroll
                for (int ii = 0; ii < 32; ii++)
                    if (32 + ii < nrows) yp[(size_t)(32 + ii) * a.H * DV] = __float2bfloat16_rn(__uint_as_float(y1[ii]));
            }
        }
    }
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
    const int smem = SM_TOTAL;
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        if (cudaFuncSetAttribute(gdn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return check_launch("gdn_prefill smem attribute");
        attr_set[dev] = true;
    }
    gdn_prefill_kernel<<<a.n_seq * a.n_heads, PF_THREADS, smem, stream>>>(tq, tk, tv, a);
    return check_launch("gdn_prefill");
}

}  // namespace gdn
