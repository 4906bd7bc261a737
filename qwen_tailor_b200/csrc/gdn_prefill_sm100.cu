// Chunked GatedDeltaNet prefill on the Blackwell tensor cores (tcgen05 / TMEM / TMA), chunk size 64, varlen batches:
// the serial chain over the chunks of one (sequence, head) -- the reference's phase B.
//
// Replaces `gdn_nax_b` / `phase_b` of the reference (qwen35/gdn_nax.py:224-358, 404-410), which steps over 16-token chunks with
// Apple simdgroup MMAs.  Same algebra (qwen35/gdn_nax.py:3-10), per head and chunk of C = 64 tokens, S0 = state entering the chunk
// ([dv, dk]), Lc = inclusive cumulative log-decay in the chunk, gamma_i = exp(Lc_i):
//     Tb = (I + L)^-1 diag(beta)                                  from phase A (gdn_phase_a.cu), with Lc, gamma, dec
//     D  = Tb (V - gamma * (K S0^T))
//     Y  = gamma * (Q S0^T) + A D,  A = lower_incl(exp(Lc_i - Lc_j) (Q K^T)_ij)
//     S1 = gamma_C S0 + D^T diag(dec) K,   dec_j = exp(Lc_C - Lc_j)
// Decay factors are always exp of a masked difference of Lc (never a ratio), so the ~1e-97 in-chunk decays of real gates
// underflow to 0 instead of producing inf * 0.
//
// Mapping.  One block = one (sequence, head) chain; the chain over chunks is serial, heads / sequences / layers are the parallel
// axis.  Every product is computed TRANSPOSED so that the 128 value rows of the head are the M dimension of a full-rate M = 128
// MMA and a TMEM lane is one value row for the whole kernel:
//     [P1^T | P2^T] [dv x 128] = S0 [K; Q]^T                            A = S0 (bf16 hi + lo) from TMEM; K and Q tiles are stacked in
//                                                                       smem, so one N = 128 product gives S0 K^T and S0 Q^T
//     G    [128 x 64]  = [K; Q] K^T            rows 64-127 = Q K^T; rows 0-63 are not used
//     D^T  [dv x 64]   = R^T Tb^T,  R^T = V^T - P1^T diag(gamma)        A = R^T (hi + lo) from TMEM (the chain warps form it in fp32)
//     YD^T [dv x 64]   = D^T A^T                                        A = D^T (hi + lo) from TMEM, B = A (hi + lo) in smem
//     S    [dv x 128] += Dp^T K,  Dp = diag(dec) D                      A = Dp^T (hi + lo) in smem, B = K read MN-major
// The fp32 state lives in TMEM for the whole sequence.  Every operand that is derived from fp32 data (S, R, D, Dp, Tb, A) is fed to
// the bf16 MMA as an exact hi + lo pair (16 significand bits), which keeps the final state within 1e-4 of fp64; K, Q and V are
// bf16 already.
//
// Roles (448 threads, one block per SM):
//   warps 0-7   "chain": the state-dependent passes between MMAs (two warps per TMEM lane quadrant, half of the columns each)
//   warps 8-11  "output": the A matrix from Q K^T, and y = gamma * P2 + YD
//   warp 12     lane 0 issues every tcgen05.mma.  An MMA instruction of this shape occupies the tensor pipe for ~90 cycles whatever
//               its N <= 128 (measured), so the kernel is bound by the NUMBER of instructions per chunk: 56 (16 for [P1 | P2],
//               8 for G, 12 for D, 8 for the state update, 12 for YD); G and YD run while the chain warps convert
//   warp 13     "producer": K / Q / V tiles by TMA (128-byte swizzle, no multicast) and the phase-A record by one bulk copy, two
//               stages; it also zeroes the rows of a partial last chunk so that a packed neighbour sequence can never leak in
// The groups hand over through mbarriers.  Two rules keep that protocol sound: every warp that waits on a barrier also takes part
// in what lets the barrier's NEXT phase complete (a waiter that fell a whole phase behind would mistake phase c + 2 for phase c,
// because only the parity is visible); and every wait is bounded -- a wait that gives up sets the device status word, tells the
// block to leave, and the block leaves after its outstanding copies have landed.
#include <cuda.h>
// waiting warps sleep ~20 ns between polls of an mbarrier: back-to-back polls take issue slots and shared-memory bandwidth from
// the warps that do the work
#define GDN_POLL_SLEEP 20
#include "gdn_common.cuh"
#include "launchers.cuh"
#include "sm100_prims.cuh"

namespace gdn {

using namespace sm100;

constexpr int CH = 64;                               // chunk length
constexpr int PB_THREADS = 448;
// ---- shared memory map (bytes from a 1024-aligned base) ----
constexpr int ST_K0 = 0, ST_Q0 = 8192, ST_K1 = 16384, ST_Q1 = 24576;      // [K_h0 | Q_h0 | K_h1 | Q_h1]: [K; Q] stacked per 64-column half
constexpr int ST_V = 32768;                          // [V_h0 | V_h1]
constexpr int ST_REC = 49152;                        // phase-A record: Tb hi, Tb lo (8 KiB each), Lc, gamma, dec ([64] fp32 each)
constexpr int ST_TB_HI = ST_REC, ST_TB_LO = ST_REC + 8192, ST_LC = ST_REC + 16384, ST_GAM = ST_LC + 256, ST_DEC = ST_GAM + 256;
constexpr int SM_STAGE = 65 * 1024;                  // 49152 + 17152 rounded up to a multiple of 1024
constexpr int SM_A_HI = 2 * SM_STAGE;                // A as bf16 hi / lo: [64][64], K-major, 8 KiB each
constexpr int SM_A_LO = SM_A_HI + 8192;
constexpr int SM_DP_HI = SM_A_LO + 8192;             // Dp^T hi / lo: [128][64] bf16, K-major, 16 KiB each
constexpr int SM_DP_LO = SM_DP_HI + 16384;
constexpr int SM_Y = SM_DP_LO + 16384;               // y tile of the chunk, [64 tokens][128 value columns] bf16, staged for row-wise stores (16 KiB)
constexpr int SM_Z = SM_Y + 16384;                    // gate rows of the chunk (fused gated norm), same shape as the y tile (16 KiB)
constexpr int SM_TOTAL = SM_Z + 16384;
static_assert(ST_DEC + 256 <= SM_STAGE && ST_DEC + 256 - ST_REC == PA_REC_BYTES, "record layout");
// ---- tensor memory map (columns) ----
constexpr uint32_t TM_S = 0;                         // fp32 state, pre-scaled by the coming chunk's gamma_C   [128 cols]
constexpr uint32_t TM_SHI = 128, TM_SLO = 192;       // bf16 pairs of the unscaled state                        [64 + 64]
constexpr uint32_t TM_X = 256;                       // [P1^T | P2^T]; once P1 has been consumed its half takes D^T  [64 + 64]
constexpr uint32_t TM_GY = 384;                      // [K;Q] K^T, later YD^T                                   [64]
constexpr uint32_t TM_ZHI = 448, TM_ZLO = 480;       // R^T, later D^T, as bf16 pairs                           [32 + 32]
// ---- mbarriers ----
enum { B_RAW0 = 0, B_RAW1, B_FULL0, B_FULL1, B_EMPTY0, B_EMPTY1, B_SREADY, B_P1DONE, B_ZREADY, B_DDONE, B_DPREADY, B_SDONE, B_GDONE, B_AREADY,
       B_YDONE, B_YFREE, B_COUNT };
constexpr int N_CHAIN_WARPS = 8, N_OUT_WARPS = 4;

constexpr uint32_t WAIT_LIMIT = 2000000u;               // polls of >= 20 ns each: tens of milliseconds before a wait gives up

__device__ __forceinline__ float ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }

__device__ __forceinline__ void split_pack(float x0, float x1, uint32_t& hi, uint32_t& lo) {
    hi = pack_bf16x2(x0, x1);
    lo = pack_bf16x2(x0 - __uint_as_float(hi << 16), x1 - __uint_as_float(hi & 0xffff0000u));
}

__device__ __forceinline__ void bulk_load_rec(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// GATED: the layer's gated RMSNorm is applied in the y store (PrefillArgs::gate_*).
template <bool GATED>
__global__ void __launch_bounds__(PB_THREADS, 1)
gdn_phase_b_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                   const PrefillArgs a) {
    // the swizzled tiles need a 1024-byte aligned base; the declared alignment provides it (checked below).  The array is used
    // directly, not through a re-aligned pointer, so that the compiler keeps every access in the shared address space
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ uint64_t bars[B_COUNT];
    __shared__ uint32_t tmem_slot;
    __shared__ int s_abort;
    __shared__ int s_group_ok[2];                                    // outcome reported by the chain / output group's polling warp on its last wait

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
        for (int i = tid * 4; i < DV * DK; i += PB_THREADS * 4)       // nothing to compute: the state passes through unchanged
            *reinterpret_cast<float4*>(fin_head + i) = init_head ? *reinterpret_cast<const float4*>(init_head + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        return;
    }
    const int nchunks = (len + CH - 1) / CH;
    const unsigned char* rec_base = a.records + ((size_t)(t_begin / CH + seq) * a.H + h) * PA_REC_BYTES;     // record of chunk 0
    const size_t rec_step = (size_t)a.H * PA_REC_BYTES;

    const uint32_t sbase = smem_addr(smem);
    if (sbase & 1023u) { if (tid == 0) atomicExch(a.status, 4); return; }
    auto bar = [&](int i) -> uint32_t { return smem_addr(&bars[i]); };
    auto stage_f = [&](int c, int off) -> const float* { return reinterpret_cast<const float*>(smem + (c & 1) * SM_STAGE + off); };

    if (tid == 0) {
        mbar_init(bar(B_RAW0), 1); mbar_init(bar(B_RAW1), 1); mbar_init(bar(B_FULL0), 1); mbar_init(bar(B_FULL1), 1);
        mbar_init(bar(B_EMPTY0), 1 + N_CHAIN_WARPS + N_OUT_WARPS); mbar_init(bar(B_EMPTY1), 1 + N_CHAIN_WARPS + N_OUT_WARPS);
        mbar_init(bar(B_SREADY), N_CHAIN_WARPS); mbar_init(bar(B_ZREADY), N_CHAIN_WARPS); mbar_init(bar(B_DPREADY), N_CHAIN_WARPS);
        mbar_init(bar(B_AREADY), N_OUT_WARPS); mbar_init(bar(B_YFREE), N_OUT_WARPS);
        mbar_init(bar(B_P1DONE), 1); mbar_init(bar(B_DDONE), 1); mbar_init(bar(B_SDONE), 1); mbar_init(bar(B_GDONE), 1); mbar_init(bar(B_YDONE), 1);
        s_abort = 0; s_group_ok[0] = 1; s_group_ok[1] = 1;
        fence_barrier_init();
        tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
    }
    if (warp == 12) { tmem_alloc(smem_addr(&tmem_slot), 512); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tb = tmem_slot;

    // one arrival per warp: every lane has already fenced its own writes, the warp barrier orders them before lane 0's arrive
    auto warp_arrive = [&](int b) {
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(b));
    };
    auto aborted = [&]() -> bool { return *(volatile int*)&s_abort != 0; };
    // a bounded wait; on failure (or when another warp has already given up) the whole block is told to leave
    auto wait = [&](int b, uint32_t parity) -> bool {
        // non-blocking polls with a short pause in between: the suspending form of the wait (try_wait) costs ~250 cycles per call on
        // this part even when the phase has long completed, which the issuing thread would pay six times per chunk
        const uint32_t addr = bar(b);
        for (uint32_t i = 0; i < WAIT_LIMIT; i++) {
            if (mbar_test_wait(addr, parity & 1u)) return true;
            if ((i & 63u) == 63u && aborted()) return false;
            __nanosleep(GDN_POLL_SLEEP);
        }
        atomicExch(&s_abort, 1);
        atomicExch(a.status, 3);
        return false;
    };
    auto wait_full = [&](int c) -> bool { return wait((c & 1) ? B_FULL1 : B_FULL0, (uint32_t)(c >> 1)); };
    // Waits of a warp group.  One warp polls the mbarrier and the others block on a hardware barrier: a polling warp takes issue
    // slots on its scheduler, and the scheduler of the MMA-issuing warp must stay free of pollers (measured: with all fourteen
    // warps polling, every wait of the issuing thread cost ~300 cycles even when its barrier had long completed).  The polling
    // warp's outcome is published before the group barrier, so the whole group takes the same exit -- a warp that left on its
    // own would strand the others at a barrier that has no timeout.
    auto chain_wait = [&](int b, uint32_t parity) -> bool {        // warps 0-7; warp 1 polls (warp 12 issues MMAs on scheduler 0)
        if (warp == 1) { const bool okw = wait(b, parity); if (lane == 0) s_group_ok[0] = okw ? 1 : 0; }
        asm volatile("bar.sync 2, 256;" ::: "memory");
        return *(volatile int*)&s_group_ok[0] != 0;
    };
    auto out_wait = [&](int b, uint32_t parity) -> bool {          // warps 8-11; warp 10 polls
        if (warp == 10) { const bool okw = wait(b, parity); if (lane == 0) s_group_ok[1] = okw ? 1 : 0; }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        return *(volatile int*)&s_group_ok[1] != 0;
    };

    if (warp < N_CHAIN_WARPS) {
        // ============================================================================================================
        // chain: the state-dependent passes between the MMAs: two warps per TMEM lane quadrant, half of the columns each
        // ============================================================================================================
        const int q = warp & 3, hf = warp >> 2;
        const int r = q * 32 + lane;                                 // value row of this thread
        const uint32_t tl = tb + ((uint32_t)(q * 32) << 16);
        bool ok = chain_wait(B_FULL0, 0);
        // ---- initial state -> TMEM: unscaled bf16 hi/lo pairs and the fp32 copy pre-scaled by gamma_C of chunk 0 ----
        if (ok) {
            const float gC0 = stage_f(0, ST_GAM)[63];
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
        for (int c = 0; ok && c < nchunks; c++) {
            const uint32_t par = (uint32_t)c;
            const bool last = c == nchunks - 1;

            // ---- R^T = V^T - P1^T diag(gamma) -> bf16 hi/lo pairs in TMEM (the A operand of R^T Tb^T) ----
            if (!chain_wait(B_P1DONE, par)) break;
            tc_fence_after_sync();
            if (warp == 0) GDN_TSTAMP(64 + c * 32 + 8);
            {
                const float* gam = stage_f(c, ST_GAM);
                // V[j][r] of the chunk's tokens j = 32 hf .. 32 hf + 31: the V tile holds rows of 64 value columns (128 bytes, swizzled
                // in 16-byte pieces), so the lanes of a warp read 64 contiguous bytes of one row
                const unsigned char* vt = smem + (c & 1) * SM_STAGE + ST_V + (r >> 6) * 8192 + (r & 7) * 2;
                const int vp = (r & 63) >> 3;
                uint32_t rr[32], hi[16], lo[16];
                tmem_ld32(tl + TM_X + hf * 32, rr);
                float vv[32];
#pragma unroll
                for (int jj = 0; jj < 32; jj++) {
                    const int j = hf * 32 + jj;
                    vv[jj] = __uint_as_float((uint32_t)*reinterpret_cast<const unsigned short*>(vt + j * 128 + ((vp ^ (j & 7)) << 4)) << 16);
                }
                tmem_wait_ld();
#pragma unroll
                for (int jj = 0; jj < 32; jj += 4) {
                    const float4 g4 = *reinterpret_cast<const float4*>(gam + hf * 32 + jj);
                    split_pack(fmaf(-g4.x, __uint_as_float(rr[jj]), vv[jj]), fmaf(-g4.y, __uint_as_float(rr[jj + 1]), vv[jj + 1]), hi[jj / 2], lo[jj / 2]);
                    split_pack(fmaf(-g4.z, __uint_as_float(rr[jj + 2]), vv[jj + 2]), fmaf(-g4.w, __uint_as_float(rr[jj + 3]), vv[jj + 3]), hi[jj / 2 + 1],
                               lo[jj / 2 + 1]);
                }
                tmem_st16(tl + TM_ZHI + hf * 16, hi);
                tmem_st16(tl + TM_ZLO + hf * 16, lo);
                tmem_wait_st();
            }
            tc_fence_before_sync();
            warp_arrive(B_ZREADY);
            if (warp == 0) GDN_TSTAMP(64 + c * 32 + 9);

            // ---- D^T -> bf16 hi/lo pairs in TMEM (A operand of D^T A^T) and Dp^T = D^T diag(dec) -> hi/lo K-major rows in smem ----
            if (!chain_wait(B_DDONE, par)) break;
            tc_fence_after_sync();
            if (warp == 0) GDN_TSTAMP(64 + c * 32 + 10);
            {
                const float* dec = stage_f(c, ST_DEC);
                uint32_t rr[32], hi[16], lo[16];
                tmem_ld32(tl + TM_X + hf * 32, rr);
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
            if (warp == 0) GDN_TSTAMP(64 + c * 32 + 11);
            warp_arrive((c & 1) ? B_EMPTY1 : B_EMPTY0);              // this warp's last read of the stage (gamma, dec) is behind it

            // ---- after the state update: bf16 hi/lo pairs of the new state for the next chunk's products, fp32 copy pre-scaled by
            //      the next chunk's gamma_C (or the final state) ----
            float gC_next = 1.f;
            if (!last) {
                if (!chain_wait(((c + 1) & 1) ? B_FULL1 : B_FULL0, (uint32_t)((c + 1) >> 1))) break;
                gC_next = stage_f(c + 1, ST_GAM)[63];
            }
            if (!chain_wait(B_SDONE, par)) break;
            tc_fence_after_sync();
            if (warp == 0) GDN_TSTAMP(64 + c * 32 + 12);
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
                if (warp == 0) GDN_TSTAMP(64 + c * 32 + 13);
            }
        }
    } else if (warp < N_CHAIN_WARPS + N_OUT_WARPS) {
        // ============================================================================================================
        // output: A from Q K^T (the two warps that own TMEM lanes 64..127) and the y rows
        // ============================================================================================================
        const int q = warp & 3;
        const int r = q * 32 + lane;
        const uint32_t tl = tb + ((uint32_t)(q * 32) << 16);
        for (int c = 0; c < nchunks; c++) {
            const uint32_t par = (uint32_t)c;
            const int t0 = t_begin + c * CH;
            const int nrows = min(CH, t_end - t0);
            if (GATED) {                                          // fused gated norm: the chunk's gate rows travel to shared memory meanwhile
                const int ot = tid - N_CHAIN_WARPS * 32;
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    const int i = (ot >> 4) + 8 * k;
                    if (i < nrows)
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sbase + SM_Z + (i * DV + (ot & 15) * 8) * 2),
                                     "l"(a.gate_z + (size_t)(t0 + i) * a.gate_stride + h * DV + (ot & 15) * 8) : "memory");
                }
                asm volatile("cp.async.commit_group;" ::: "memory");
            }
            if (!out_wait((c & 1) ? B_FULL1 : B_FULL0, (uint32_t)(c >> 1))) break;      // Lc and gamma of the chunk have landed
            // ---- A = lower_incl(exp(Lc_i - Lc_j) Q K^T) as bf16 hi/lo K-major rows (the previous chunk's D^T A^T has completed) ----
            if (!out_wait(B_GDONE, par)) break;
            tc_fence_after_sync();
            if (q >= 2) {
                const int i = r - 64;
                const float* Lc = stage_f(c, ST_LC);
                const float Li = Lc[i];
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    uint32_t rr[32];
                    tmem_ld32(tl + TM_GY + half * 32, rr);
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
            }
            tc_fence_before_sync();
            warp_arrive(B_AREADY);                                   // all four warps: each of them waited on B_GDONE (see the rule above)
            // ---- y[t0 + i, h, v] = gamma_i P2^T[v][i] + YD^T[v][i]: each lane owns one value row, a warp store covers 64 contiguous bytes ----
            if (!out_wait(B_YDONE, par)) break;
            tc_fence_after_sync();
            if (warp == 8) GDN_TSTAMP(64 + c * 32 + 14);
            {
                const float* gam = stage_f(c, ST_GAM);
                uint32_t ya[32], yb[32];
                {
                    uint32_t yd[32];
                    tmem_ld32(tl + TM_X + 64, ya);
                    tmem_ld32(tl + TM_GY, yd);
                    tmem_wait_ld();
#pragma unroll
                    for (int ii = 0; ii < 32; ii += 4) {
                        const float4 g4 = *reinterpret_cast<const float4*>(gam + ii);
                        ya[ii] = __float_as_uint(fmaf(g4.x, __uint_as_float(ya[ii]), __uint_as_float(yd[ii])));
                        ya[ii + 1] = __float_as_uint(fmaf(g4.y, __uint_as_float(ya[ii + 1]), __uint_as_float(yd[ii + 1])));
                        ya[ii + 2] = __float_as_uint(fmaf(g4.z, __uint_as_float(ya[ii + 2]), __uint_as_float(yd[ii + 2])));
                        ya[ii + 3] = __float_as_uint(fmaf(g4.w, __uint_as_float(ya[ii + 3]), __uint_as_float(yd[ii + 3])));
                    }
                    tmem_ld32(tl + TM_X + 96, yb);
                    tmem_ld32(tl + TM_GY + 32, yd);
                    tmem_wait_ld();
                    tc_fence_before_sync();
                    warp_arrive(B_YFREE);                            // the columns may take the next chunk's products
#pragma unroll
                    for (int ii = 0; ii < 32; ii += 4) {
                        const float4 g4 = *reinterpret_cast<const float4*>(gam + 32 + ii);
                        yb[ii] = __float_as_uint(fmaf(g4.x, __uint_as_float(yb[ii]), __uint_as_float(yd[ii])));
                        yb[ii + 1] = __float_as_uint(fmaf(g4.y, __uint_as_float(yb[ii + 1]), __uint_as_float(yd[ii + 1])));
                        yb[ii + 2] = __float_as_uint(fmaf(g4.z, __uint_as_float(yb[ii + 2]), __uint_as_float(yd[ii + 2])));
                        yb[ii + 3] = __float_as_uint(fmaf(g4.w, __uint_as_float(yb[ii + 3]), __uint_as_float(yd[ii + 3])));
                    }
                }
                warp_arrive((c & 1) ? B_EMPTY1 : B_EMPTY0);          // gamma was this warp's last read of the stage
                const int ot = tid - N_CHAIN_WARPS * 32;             // 0..127: row (ot >> 4) + 8 k, 16-byte word ot & 15 of the y tile
                // transpose through shared memory: a lane owns one value column of all 64 tokens, the rows of y want 256 contiguous bytes
                __nv_bfloat16* ys = reinterpret_cast<__nv_bfloat16*>(smem + SM_Y);
                unsigned short* ysu = reinterpret_cast<unsigned short*>(ys);
#pragma unroll
                for (int ii = 0; ii < 32; ii += 2) {                 // packed conversions (two tokens at a time), 16-bit stores
                    const uint32_t pa = pack_bf16x2(__uint_as_float(ya[ii]), __uint_as_float(ya[ii + 1]));
                    const uint32_t pb = pack_bf16x2(__uint_as_float(yb[ii]), __uint_as_float(yb[ii + 1]));
                    ysu[ii * DV + r] = (unsigned short)pa;
                    ysu[(ii + 1) * DV + r] = (unsigned short)(pa >> 16);
                    ysu[(32 + ii) * DV + r] = (unsigned short)pb;
                    ysu[(33 + ii) * DV + r] = (unsigned short)(pb >> 16);
                }
                if (GATED) asm volatile("cp.async.wait_group 0;" ::: "memory");      // this thread's part of the gate rows has landed
                asm volatile("bar.sync 1, 128;" ::: "memory");       // the four output warps
                if (!GATED) {
#pragma unroll
                    for (int k = 0; k < 8; k++) {
                        const int p = ot + 128 * k, i = p >> 4, c16 = p & 15;
                        if (i < nrows)
                            *reinterpret_cast<uint4*>(a.y + ((size_t)(t0 + i) * a.H + h) * DV + c16 * 8) = *reinterpret_cast<const uint4*>(ys + i * DV + c16 * 8);
                    }
                } else {
                    // gated RMSNorm on the bf16 y rows (the stand-alone kernel's arithmetic, gnorm_* in gdn_common.cuh): sixteen
                    // threads share a row, each with eight of its values = two of that kernel's groups of four
                    const int c16 = ot & 15;
                    // pass 1: the eight rows' sums of squares, their shuffle chains side by side
                    float inv[8];
#pragma unroll
                    for (int k = 0; k < 8; k++) {
                        const uint4 yr = *reinterpret_cast<const uint4*>(ys + ((ot >> 4) + 8 * k) * DV + c16 * 8);
                        float yy[8];
                        unpack_bf16x4(make_uint2(yr.x, yr.y), yy);
                        unpack_bf16x4(make_uint2(yr.z, yr.w), yy + 4);
                        inv[k] = gnorm_sq4(yy) + gnorm_sq4(yy + 4);
                    }
#pragma unroll
                    for (int o = 1; o < 16; o <<= 1) {
#pragma unroll
                        for (int k = 0; k < 8; k++) inv[k] += __shfl_xor_sync(0xffffffffu, inv[k], o);
                    }
#pragma unroll
                    for (int k = 0; k < 8; k++) inv[k] = gnorm_inv(inv[k]);
                    float gw8[8];                                    // the norm weights of this thread's eight columns
                    *reinterpret_cast<float4*>(gw8) = __ldg(reinterpret_cast<const float4*>(a.gate_w + c16 * 8));
                    *reinterpret_cast<float4*>(gw8 + 4) = __ldg(reinterpret_cast<const float4*>(a.gate_w + c16 * 8 + 4));
                    // pass 2: the elements
#pragma unroll
                    for (int k = 0; k < 8; k++) {
                        const int i = (ot >> 4) + 8 * k;
                        const uint4 yr = *reinterpret_cast<const uint4*>(ys + i * DV + c16 * 8);
                        float yy[8], zz[8];
                        unpack_bf16x4(make_uint2(yr.x, yr.y), yy);
                        unpack_bf16x4(make_uint2(yr.z, yr.w), yy + 4);
                        const uint4 zr = *reinterpret_cast<const uint4*>(smem + SM_Z + (i * DV + c16 * 8) * 2);      // (written by this thread)
                        unpack_bf16x4(make_uint2(zr.x, zr.y), zz);
                        unpack_bf16x4(make_uint2(zr.z, zr.w), zz + 4);
                        float r8[8];
#pragma unroll
                        for (int e = 0; e < 8; e++) r8[e] = gnorm_elem(zz[e], yy[e], inv[k], gw8[e]);
                        uint4 pk;
                        pk.x = pack_bf16x2(r8[0], r8[1]); pk.y = pack_bf16x2(r8[2], r8[3]);
                        pk.z = pack_bf16x2(r8[4], r8[5]); pk.w = pack_bf16x2(r8[6], r8[7]);
                        if (i < nrows) *reinterpret_cast<uint4*>(a.y + ((size_t)(t0 + i) * a.H + h) * DV + c16 * 8) = pk;
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");       // the tile may be overwritten by the next chunk
            }
            if (warp == 8) GDN_TSTAMP(64 + c * 32 + 15);
        }
    } else if (warp == 12) {
        // ============================================================================================================
        // the MMA issuer (one thread)
        // ============================================================================================================
        if (lane == 0) {
            constexpr uint32_t I64 = idesc_bf16(128, 64, 0, 0);      // N = 64, A and B K-major (A may also come from TMEM)
            constexpr uint32_t I128 = idesc_bf16(128, 128, 0, 0);    // N = 128: B = the stacked [K; Q] rows
            constexpr uint32_t I128_BMN = idesc_bf16(128, 128, 0, 1);// N = 128, B read MN-major (K as the [tokens x dk] factor)
            for (int c = 0; c < nchunks; c++) {
                const uint32_t par = (uint32_t)c;
                const uint32_t st = sbase + (c & 1) * SM_STAGE;
                if (aborted()) break;
                // ---- [P1^T | P2^T] = S0 [K; Q]^T (S0 = hi + lo from TMEM).  The accumulator columns held the previous chunk's P2^T and
                //      D^T; the G / YD columns its YD^T: both are free once the output warps have read that chunk's y ----
                if (!wait_full(c)) break;
                GDN_TSTAMP(64 + c * 32 + 16);
                if (!wait(B_SREADY, par)) break;
                GDN_TSTAMP(64 + c * 32 + 17);
                if (c >= 1 && !wait(B_YFREE, par - 1)) break;
                tc_fence_after_sync();
                GDN_TSTAMP(64 + c * 32 + 0);
#pragma unroll
                for (int part = 0; part < 2; part++) {
                    const uint32_t acol = part ? TM_SLO : TM_SHI;
#pragma unroll
                    for (int ks = 0; ks < 8; ks++) {
                        const uint32_t off = (ks >> 2) * 16384 + (ks & 3) * 32;
                        mma_ts(tb + TM_X, tb + acol + ks * 8, smem_desc_sw128(st + ST_K0 + off, 16, 1024), I128, (part | ks) != 0);
                    }
                }
                mma_commit(bar(B_P1DONE));
                GDN_TSTAMP(64 + c * 32 + 1);
                // ---- G = [K; Q] K^T: state-independent, runs while the chain warps form R ----
#pragma unroll
                for (int ks = 0; ks < 8; ks++) {
                    const uint32_t off = (ks >> 2) * 16384 + (ks & 3) * 32;
                    const uint64_t d = smem_desc_sw128(st + off, 16, 1024);
                    mma_ss(tb + TM_GY, d, d, I64, ks > 0);
                }
                mma_commit(bar(B_GDONE));
                // ---- D^T = R^T Tb^T over the columns P1 has left ----
                if (!wait(B_ZREADY, par)) break;
                tc_fence_after_sync();
                GDN_TSTAMP(64 + c * 32 + 2);
#pragma unroll
                for (int term = 0; term < 3; term++) {
                    const uint32_t acol = term == 1 ? TM_ZLO : TM_ZHI;
                    const uint32_t bsm = st + (term == 2 ? ST_TB_LO : ST_TB_HI);
#pragma unroll
                    for (int ks = 0; ks < 4; ks++)
                        mma_ts(tb + TM_X, tb + acol + ks * 8, smem_desc_sw128(bsm + ks * 32, 16, 1024), I64, (term | ks) != 0);
                }
                mma_commit(bar(B_DDONE));
                GDN_TSTAMP(64 + c * 32 + 3);
                // ---- the state update S += Dp^T K ----
                if (!wait(B_DPREADY, par)) break;
                tc_fence_after_sync();
                GDN_TSTAMP(64 + c * 32 + 4);
#pragma unroll
                for (int part = 0; part < 2; part++) {
                    const uint32_t asm_ = sbase + (part ? SM_DP_LO : SM_DP_HI);
#pragma unroll
                    for (int ks = 0; ks < 4; ks++)
                        mma_ss(tb + TM_S, smem_desc_sw128(asm_ + ks * 32, 16, 1024), smem_desc_sw128(st + ST_K0 + ks * 2048, 16384, 1024), I128_BMN, 1);
                }
                mma_commit(bar(B_SDONE));
                GDN_TSTAMP(64 + c * 32 + 5);
                // ---- YD^T = D^T A^T over the columns G has left ----
                if (!wait(B_AREADY, par)) break;
                tc_fence_after_sync();
                GDN_TSTAMP(64 + c * 32 + 6);
#pragma unroll
                for (int term = 0; term < 3; term++) {
                    const uint32_t acol = term == 1 ? TM_ZLO : TM_ZHI;
                    const uint32_t bsm = sbase + (term == 2 ? SM_A_LO : SM_A_HI);
#pragma unroll
                    for (int ks = 0; ks < 4; ks++) mma_ts(tb + TM_GY, tb + acol + ks * 8, smem_desc_sw128(bsm + ks * 32, 16, 1024), I64, (term | ks) != 0);
                }
                mma_commit(bar(B_YDONE));
                GDN_TSTAMP(64 + c * 32 + 7);
                mma_commit(bar((c & 1) ? B_EMPTY1 : B_EMPTY0));      // every MMA that reads this stage has completed when this arrives
            }
        }
    } else {
        // ============================================================================================================
        // producer: tile and record copies, two stages
        // ============================================================================================================
        int issued = 0, landed = 0;
        auto issue = [&](int c) {                                    // lane 0: K, Q, V tiles and the phase-A record of chunk c -> stage c & 1
            const uint32_t st = sbase + (c & 1) * SM_STAGE;
            const uint32_t kb = bar((c & 1) ? B_RAW1 : B_RAW0);
            const int t0 = t_begin + c * CH;
            mbar_expect_tx(kb, 6 * 8192 + PA_REC_BYTES);
            tma_load_3d(st + ST_K0, &tmK, kb, 0, h, t0);
            tma_load_3d(st + ST_Q0, &tmQ, kb, 0, h, t0);
            tma_load_3d(st + ST_K1, &tmK, kb, 64, h, t0);
            tma_load_3d(st + ST_Q1, &tmQ, kb, 64, h, t0);
            tma_load_3d(st + ST_V, &tmV, kb, 0, h, t0);
            tma_load_3d(st + ST_V + 8192, &tmV, kb, 64, h, t0);
            bulk_load_rec(st + ST_REC, rec_base + (size_t)c * rec_step, PA_REC_BYTES, kb);
        };
        if (lane == 0) { issue(0); if (nchunks > 1) issue(1); }
        issued = min(nchunks, 2);
        for (int c = 0; c < nchunks; c++) {
            if (aborted()) break;
            if (!wait((c & 1) ? B_RAW1 : B_RAW0, (uint32_t)(c >> 1))) break;
            landed = c + 1;
            const int nrows = min(CH, t_end - (t_begin + c * CH));
            if (nrows < CH) {
                // rows past the end of the sequence are zero (qwen35/gdn_nax.py:55-60): 6 tiles x (64 - nrows) rows x 128 B
                const int nz = (CH - nrows) * 8;
                for (int i = lane; i < 6 * nz; i += 32) {
                    const int tile = i / nz, p = i % nz;
                    *reinterpret_cast<uint4*>(smem + (c & 1) * SM_STAGE + tile * 8192 + nrows * 128 + p * 16) = make_uint4(0, 0, 0, 0);
                }
                fence_proxy_async_smem();
            }
            warp_arrive((c & 1) ? B_FULL1 : B_FULL0);
            // refill the other stage (chunk c + 1 lives there only if c >= 1: chunks 0 and 1 were issued up front)
            if (c >= 1 && c + 1 < nchunks) {
                if (!wait(((c + 1) & 1) ? B_EMPTY1 : B_EMPTY0, (uint32_t)((c - 1) >> 1))) break;
                if (lane == 0) issue(c + 1);
                issued = c + 2;
            }
        }
        // leaving early: the copies that were issued must land before the block's shared memory is given up
        for (int c = landed; c < issued; c++) wait((c & 1) ? B_RAW1 : B_RAW0, (uint32_t)(c >> 1));
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 12) tmem_dealloc(tb, 512);
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
int make_token_map(CUtensorMap* m, const void* base, long long total_T, int H) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) { set_error("gdn prefill: cuTensorMapEncodeTiled is not available from this driver"); return GDN_E_UNSUPPORTED; }
    const cuuint64_t dims[3] = {128, (cuuint64_t)H, (cuuint64_t)total_T};
    const cuuint64_t strides[2] = {256, (cuuint64_t)H * 256};
    const cuuint32_t box[3] = {64, 1, 64}, es[3] = {1, 1, 1};
    const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("gdn prefill: cuTensorMapEncodeTiled failed with code %d", (int)r); return GDN_E_LAUNCH; }
    return GDN_OK;
}

int launch_phase_b(const void* q, const void* k, const void* v, const PrefillArgs& a, cudaStream_t stream) {
    if (a.n_seq <= 0 || a.n_heads <= 0) return GDN_OK;
    CUtensorMap tq, tk, tv;
    int rc;
    if ((rc = make_token_map(&tq, q, a.total_T, a.H)) || (rc = make_token_map(&tk, k, a.total_T, a.H)) || (rc = make_token_map(&tv, v, a.total_T, a.H)))
        return rc;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    const int smem = SM_TOTAL;
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        if (cudaFuncSetAttribute(gdn_phase_b_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess ||
            cudaFuncSetAttribute(gdn_phase_b_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return check_launch("gdn_phase_b smem attribute");
        attr_set[dev] = true;
    }
    if (a.gate_w) gdn_phase_b_kernel<true><<<a.n_seq * a.n_heads, PB_THREADS, smem, stream>>>(tq, tk, tv, a);
    else gdn_phase_b_kernel<false><<<a.n_seq * a.n_heads, PB_THREADS, smem, stream>>>(tq, tk, tv, a);
    return check_launch("gdn_phase_b");
}

}  // namespace gdn

#ifdef GDN_TIMING
extern "C" __attribute__((visibility("default"))) int gdn_timing_log_b(long long* out_host, int n) {
    return cudaMemcpyFromSymbol(out_host, gdn::g_tlog, sizeof(long long) * n) == cudaSuccess ? 0 : -5;
}
#endif
