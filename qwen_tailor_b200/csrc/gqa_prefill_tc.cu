// Causal prefill attention, head_dim 256, GQA 8 query heads on 2 KV heads, on the Blackwell tensor cores (tcgen05 / TMEM / TMA).
//
// Replaces the scaled-dot-product call of the reference's prefill (qwen35/model.py:148-169, the `mx.fast.scaled_dot_product_attention`
// at :165, reached from qwen35/prefill.py:468): for the S query tokens at positions pos .. pos + S - 1,
//     o[i, h, :] = softmax(q[i, h, :] . K[0 .. pos + i, h / 4, :] / 16) V[0 .. pos + i, h / 4, :]
// with bf16 inputs and output and fp32 scores, sums and accumulation.
//
// One block per (KV head, 32 query tokens): the 4 query heads that share the KV head and the 32 tokens make the 128 rows of the
// tensor-core tile (row = token * 4 + head), so a K / V tile is read once for four heads.  Per 128-key tile:
//     S [128 x 128]  = Q K^T        16 MMAs (K = 256 dims, N = 128), A = Q (shared memory, loaded once), B = K slabs as TMA wrote them
//     P              = 2^(S sc - m) one thread per row (no cross-lane reduction), bf16 hi + lo pairs written over the scores
//     O [128 x 256] += P V          16 MMAs (K = 128 keys, hi and lo), A = P from tensor memory, B = V chunks read N-major
// Two score / P buffers of 128 columns next to the 256 columns of O fill the tensor memory: the softmax of tile t runs while the
// tensor pipe forms the scores of tile t + 1 and the P V product of tile t - 1.  The running maximum is only raised when a tile
// exceeds it by more than 2^8, so the rescale of O (a round trip through registers) is rare; l and O carry the same reference, so
// the result does not depend on it.  Blocks are numbered so that the ones with the most keys (the last query tokens) start first.
//
// Roles (192 threads): warps 0-3 softmax / epilogue (thread = row = TMEM lane), warp 4 lane 0 issues the MMAs, warp 5 lane 0 is the
// TMA producer: Q once (64 KiB), then K in slabs of 64 dims and V in chunks of 32 keys (16 KiB each) through two five-slot rings,
// a slot being refilled as soon as the four MMAs that read it are done.  Measured: a tile takes ~5.7 k cycles against 3.8 k of MMA
// issue; per tile 384 KiB cross the SM's shared-memory port (Q and K operands of the score MMAs, V once for hi and once for lo, the
// TMA writes), which at 128 B per cycle is 3 k cycles of its own.
// Optionally (workspace given) the query blocks with the most keys run as two blocks along the keys that leave (O, m, l) partials
// and are merged by the one that arrives last.
// Every wait is bounded; a wait that gives up sets the device status word and the block runs out its loops without touching the
// tensor cores again.
#include <cuda.h>
#include <cstring>
#include "gdn_common.cuh"
#include "gqa_common.cuh"
#include "sm100_prims.cuh"

namespace gdn {

using namespace sm100;

constexpr int PF_THREADS = 192;
constexpr int PF_QTOK = 32;                                          // query tokens per block (x 4 heads = 128 rows)
constexpr int PF_TK = 128;                                           // keys per tile
constexpr int PF_Q_BYTES = 128 * ATT_D * 2;                          // 64 KiB: 4 slabs of [128 rows][64 dims]
constexpr int PF_SLOT = 16384;                                       // a K slab [128 keys][64 dims] or a V chunk [32 keys][256 dims]
constexpr int PF_NK = 5, PF_NV = 5;                                  // ring slots of K slabs and of V chunks
constexpr int PF_SMEM = PF_Q_BYTES + (PF_NK + PF_NV) * PF_SLOT;      // 224 KiB
constexpr uint32_t PFM_O = 0, PFM_SP0 = 256;                         // O [256], two buffers of 128 columns: scores, then P in their place
enum { PB_QFULL = 0, PB_KFULL0 = 1, PB_KEMPTY0 = PB_KFULL0 + PF_NK, PB_VFULL0 = PB_KEMPTY0 + PF_NK, PB_VEMPTY0 = PB_VFULL0 + PF_NV,
       PB_SDONE0 = PB_VEMPTY0 + PF_NV, PB_PREADY0 = PB_SDONE0 + 2, PB_PFREE0 = PB_PREADY0 + 2, PB_ODONE = PB_PFREE0 + 2, PB_COUNT };
constexpr float PF_RESCALE_STEP = 8.f;                               // log2 units

struct PrefillAttnArgs {
    __nv_bfloat16* out;        // [S, 8, 256]
    int S, pos;                // query tokens and the position of the first one; keys 0 .. pos + S - 1 exist
    int kv_head_major;         // K / V are [2, T, 256] (the tensor maps then order their dimensions (256, T, 2)) instead of [T, 2, 256]
    int heavy_tiles;           // query blocks with at least this many key tiles are split into two blocks along the keys (0: never)
    unsigned char* ws;         // workspace of the split blocks: arrival counters, then one partial (O, m, l) per (block, half)
    int* status;
};
constexpr int PF_PART_FLOATS = 128 * (ATT_D + 4);                    // a partial: [128 rows][256 O | m | l | pad 2] fp32 (rows 16-byte aligned)
constexpr int PF_WS_HEADER = 16;                                     // bytes: the epoch word
__host__ __device__ inline int pf_tiles_of(int qb, int S, int pos) { return (pos + min(PF_QTOK * (qb + 1), S) - 1) / PF_TK + 1; }

__global__ void __launch_bounds__(PF_THREADS, 1)
gqa_prefill_tc_kernel(const PrefillAttnArgs a, const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV) {
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ uint64_t bars[PB_COUNT];
    __shared__ uint32_t tmem_slot;
    __shared__ int s_abort, s_last;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t sbase = smem_addr(smem);
    if (sbase & 1023u) { if (tid == 0) atomicExch(a.status, 4); return; }
    // Work items, most keys first: the query blocks with at least `heavy_tiles` key tiles (the last ones: the tile count grows with
    // the position) are split in two along the keys -- four items per such query block (2 KV heads x 2 halves) -- then the others.
    const int n_qb = (a.S + PF_QTOK - 1) / PF_QTOK;
    int q_heavy = n_qb;                                              // first heavy query block
    if (a.heavy_tiles > 0) {
        int l = 0, r = n_qb;                                         // tiles_of is non-decreasing in the query block
        while (l < r) { const int m = (l + r) >> 1; if (pf_tiles_of(m, a.S, a.pos) >= a.heavy_tiles) r = m; else l = m + 1; }
        q_heavy = l;
    }
    const int n_heavy_items = 4 * (n_qb - q_heavy);
    int qb, kvh, part = 0, nparts = 1, unit = 0;
    if ((int)blockIdx.x < n_heavy_items) {
        unit = (int)blockIdx.x >> 1; part = (int)blockIdx.x & 1; nparts = 2;
        qb = n_qb - 1 - (unit >> 1); kvh = unit & 1;
    } else {
        const int j = (int)blockIdx.x - n_heavy_items;
        qb = q_heavy - 1 - (j >> 1); kvh = j & 1;
    }
    const int tok0 = qb * PF_QTOK;                                   // first query token of the block (relative to the call)
    const int all_tiles = pf_tiles_of(qb, a.S, a.pos);               // tiles up to the last key any row of the block sees
    const int tile0 = part == 0 ? 0 : all_tiles / 2;                 // this item's tiles: [tile0, tile0 + ntiles)
    const int ntiles = nparts == 1 ? all_tiles : (part == 0 ? all_tiles / 2 : all_tiles - all_tiles / 2);

    auto bar = [&](int i) -> uint32_t { return smem_addr(&bars[i]); };
    if (tid == 0) {
        mbar_init(bar(PB_QFULL), 1);
        for (int i = 0; i < PF_NK; i++) { mbar_init(bar(PB_KFULL0 + i), 1); mbar_init(bar(PB_KEMPTY0 + i), 1); }
        for (int i = 0; i < PF_NV; i++) { mbar_init(bar(PB_VFULL0 + i), 1); mbar_init(bar(PB_VEMPTY0 + i), 1); }
        for (int i = 0; i < 2; i++) { mbar_init(bar(PB_SDONE0 + i), 1); mbar_init(bar(PB_PREADY0 + i), 4); mbar_init(bar(PB_PFREE0 + i), 1); }
        mbar_init(bar(PB_ODONE), 1);
        s_abort = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
    }
    if (warp == 4) { tmem_alloc(smem_addr(&tmem_slot), 512); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tb = tmem_slot;

    auto aborted = [&]() -> bool { return *(volatile int*)&s_abort != 0; };
    auto wait = [&](int b, uint32_t parity) -> bool {                // bounded; a failure tells the whole block to stop computing
        const uint32_t addr = bar(b);
        for (uint32_t i = 0; i < 2000000u; i++) {
            if (mbar_test_wait(addr, parity & 1u)) return true;
            if ((i & 63u) == 63u && aborted()) return false;
            __nanosleep(20);
        }
        atomicExch(&s_abort, 1);
        atomicExch(a.status, 2);
        return false;
    };
    const uint32_t sQ = sbase, sK = sbase + PF_Q_BYTES, sV = sK + PF_NK * PF_SLOT;
    // Arrival counters of the split blocks (workspace): 64-bit words {tag, count}, valid only while the tag is the one of this call's
    // epoch; the block that leaves the kernel last advances the epoch word, which invalidates every counter at once, so nothing has to
    // be zeroed between calls and whatever an allocator left in the workspace reads as "no arrivals yet".  A block `touch`es a counter
    // long before it arrives at it: if the word is stale, one compare-and-swap (whoever wins) makes it {tag, 0}.
    const int n_split_units = n_heavy_items / 2;
    const size_t ws_parts_off = (size_t)PF_WS_HEADER + 8 * (size_t)(1 + n_split_units);      // (a multiple of 8; partials need 16)
    const size_t ws_parts_off16 = (ws_parts_off + 15) & ~(size_t)15;
    uint32_t epoch = 0;
    unsigned long long* counters = nullptr;
    if (n_split_units > 0) {
        epoch = *reinterpret_cast<volatile uint32_t*>(a.ws);
        counters = reinterpret_cast<unsigned long long*>(a.ws + PF_WS_HEADER);
    }
    auto tag_of = [&](int idx) -> uint32_t { return epoch * 0x9E3779B1u + (uint32_t)idx + 1u; };
    auto touch = [&](int idx) {
        const unsigned long long v = *reinterpret_cast<volatile unsigned long long*>(counters + idx);
        if ((uint32_t)(v >> 32) != tag_of(idx)) atomicCAS(counters + idx, v, (unsigned long long)tag_of(idx) << 32);
    };
    auto arrive = [&](int idx) -> uint32_t { return (uint32_t)atomicAdd(counters + idx, 1ull); };      // how many arrived before
    if (tid == 0 && n_split_units > 0) { touch(0); if (nparts == 2) touch(1 + unit); }

    if (warp == 5) {
        // ================= producer =================
        // K travels in slabs of 64 dims (what four of a tile's sixteen score MMAs read), V in chunks of 32 keys (what four of its
        // sixteen P V MMAs read), each through its own ring: a slot is refilled as soon as those four MMAs are done.  The copies are
        // issued in the order of use: K of tile n + 1, then V of tile n.
        if (lane == 0) {
            mbar_expect_tx(bar(PB_QFULL), PF_Q_BYTES);
            for (int j = 0; j < 4; j++) tma_load_3d(sQ + j * 16384, &tmQ, bar(PB_QFULL), 64 * j, kvh * ATT_GQA, tok0);
            uint32_t nk = 0, nv = 0;                                 // slabs / chunks issued so far
            auto load_k = [&](int n) -> bool {
                for (int j = 0; j < 4; j++, nk++) {
                    const int slot = nk % PF_NK;
                    if (nk >= (uint32_t)PF_NK && !wait(PB_KEMPTY0 + slot, nk / PF_NK - 1)) return false;
                    mbar_expect_tx(bar(PB_KFULL0 + slot), PF_SLOT);
                    tma_load_3d(sK + slot * PF_SLOT, &tmK, bar(PB_KFULL0 + slot), 64 * j, a.kv_head_major ? (tile0 + n) * PF_TK : kvh, a.kv_head_major ? kvh : (tile0 + n) * PF_TK);
                }
                return true;
            };
            auto load_v = [&](int n) -> bool {
                for (int c = 0; c < 4; c++, nv++) {
                    const int slot = nv % PF_NV;
                    if (nv >= (uint32_t)PF_NV && !wait(PB_VEMPTY0 + slot, nv / PF_NV - 1)) return false;
                    mbar_expect_tx(bar(PB_VFULL0 + slot), PF_SLOT);
                    const int key = (tile0 + n) * PF_TK + 32 * c;
                    for (int j = 0; j < 4; j++)
                        tma_load_3d(sV + slot * PF_SLOT + j * 4096, &tmV, bar(PB_VFULL0 + slot), 64 * j, a.kv_head_major ? key : kvh, a.kv_head_major ? kvh : key);
                }
                return true;
            };
            bool okp = load_k(0);
            for (int n = 0; n < ntiles && okp; n++) {
                if (n + 1 < ntiles) okp = load_k(n + 1);
                if (okp) okp = load_v(n);
            }
        }
    } else if (warp == 4) {
        // ================= MMA issuer =================
        if (lane == 0) {
            constexpr uint32_t I_QK = idesc_bf16(128, 128, 0, 0);
            constexpr uint32_t I_PV = idesc_bf16(128, 256, 0, 1);    // B = V read N-major (dims contiguous)
            constexpr uint32_t HI = smem_desc_hi_sw128(1024);
            uint32_t nk = 0, nv = 0;                                 // slabs / chunks consumed so far
            auto issue_pv = [&](int m) -> bool {
                const uint32_t sp = tb + PFM_SP0 + (m & 1) * 128;
                if (!wait(PB_PREADY0 + (m & 1), (uint32_t)(m >> 1))) return false;
                for (int c = 0; c < 4; c++, nv++) {                  // chunk c = keys 32 c .. 32 c + 31 = columns [32 c, 32 c + 32) of the buffer
                    const int slot = nv % PF_NV;
                    if (!wait(PB_VFULL0 + slot, nv / PF_NV)) return false;
                    tc_fence_after_sync();
                    const uint32_t vlo = smem_desc_lo(sV + slot * PF_SLOT, 4096);
                    for (int part = 0; part < 2; part++)             // hi, lo
                        for (int ks = 0; ks < 2; ks++) {
                            const uint32_t acol = sp + 32 * c + 16 * part + 8 * ks;
                            if (m == 0 && c == 0 && part == 0 && ks == 0) mma_ts_w<false>(tb + PFM_O, acol, vlo + ks * 128, HI, I_PV);
                            else mma_ts_w<true>(tb + PFM_O, acol, vlo + ks * 128, HI, I_PV);
                        }
                    mma_commit(bar(PB_VEMPTY0 + slot));
                }
                mma_commit(bar(PB_PFREE0 + (m & 1)));
                return true;
            };
            bool ok = wait(PB_QFULL, 0);
            const uint32_t qlo = smem_desc_lo(sQ, 16);
            for (int n = 0; n < ntiles && ok && !aborted(); n++) {
                // the buffer of tile n held P of tile n - 2: its P V product was issued before this point and the tensor pipe runs
                // the MMAs of one thread in the order of issue, so these scores cannot overtake it
                const uint32_t sp = tb + PFM_SP0 + (n & 1) * 128;
                for (int j = 0; j < 4 && ok; j++, nk++) {
                    const int slot = nk % PF_NK;
                    if (!wait(PB_KFULL0 + slot, nk / PF_NK)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t klo = smem_desc_lo(sK + slot * PF_SLOT, 16);
#pragma unroll
                    for (int kk = 0; kk < 4; kk++) {
                        if (j == 0 && kk == 0) mma_ss_w<false>(sp, qlo + j * (16384 >> 4) + kk * 2, HI, klo + kk * 2, HI, I_QK);
                        else mma_ss_w<true>(sp, qlo + j * (16384 >> 4) + kk * 2, HI, klo + kk * 2, HI, I_QK);
                    }
                    mma_commit(bar(PB_KEMPTY0 + slot));
                }
                if (!ok) break;
                mma_commit(bar(PB_SDONE0 + (n & 1)));
                GDN_TSTAMP(n * 8 + 0);
                if (n >= 1) ok = issue_pv(n - 1);
                GDN_TSTAMP(n * 8 + 1);
            }
            if (ok && !aborted()) ok = issue_pv(ntiles - 1);
            if (ok) mma_commit(bar(PB_ODONE));
        }
    } else {
        // ================= softmax and epilogue: thread = row = token * 4 + head =================
        const float sc = 0.0625f * 1.4426950408889634f;              // 256^-1/2, scores kept in log2 units
        const int row = warp * 32 + lane;
        const int tok = tok0 + (row >> 2);                           // query token of this row (relative to the call)
        const int my_pos = a.pos + tok;                              // keys 0 .. my_pos are visible
        const uint32_t tl = tb + ((uint32_t)(warp * 32) << 16);      // this warp's TMEM lanes
        float m_run = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (int n = 0; n < ntiles && ok; n++) {
            const uint32_t sp = tl + PFM_SP0 + (n & 1) * 128;
            if (!wait(PB_SDONE0 + (n & 1), (uint32_t)(n >> 1))) { ok = false; break; }
            tc_fence_after_sync();
            if (warp == 0) GDN_TSTAMP(n * 8 + 2);
            const int key0 = (tile0 + n) * PF_TK;
            const bool masked = key0 + PF_TK - 1 > a.pos + tok0;     // the tile reaches past the block's first query: causal mask
            // the row's 128 scores (four loads in flight, one wait), masked, and their maximum
            float sv[128];
            {
                uint32_t r0[32], r1[32], r2[32], r3[32];
                tmem_ld32(sp, r0); tmem_ld32(sp + 32, r1); tmem_ld32(sp + 64, r2); tmem_ld32(sp + 96, r3);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    sv[i] = __uint_as_float(r0[i]); sv[32 + i] = __uint_as_float(r1[i]);
                    sv[64 + i] = __uint_as_float(r2[i]); sv[96 + i] = __uint_as_float(r3[i]);
                }
            }
            if (masked) {
#pragma unroll
                for (int i = 0; i < 128; i++) sv[i] = (key0 + i <= my_pos) ? sv[i] : -INFINITY;
            }
            float mt = -INFINITY;
#pragma unroll
            for (int i = 0; i < 128; i += 4) mt = fmaxf(mt, fmaxf(fmaxf(sv[i], sv[i + 1]), fmaxf(sv[i + 2], sv[i + 3])));
            if (warp == 0) GDN_TSTAMP(n * 8 + 3);
            mt *= sc;                                                // (sc > 0: the maximum of the scaled scores)
            // raise the reference only when it is far behind (or not set yet); O is rescaled then -- all lanes take part in the
            // tensor-memory round trip, each with its own factor
            const bool raise = mt > m_run + PF_RESCALE_STEP || (m_run == -INFINITY && mt != -INFINITY);
            if (__any_sync(0xffffffffu, raise)) {
                const float m_new = raise ? mt : m_run;
                const float alpha = (m_run == -INFINITY) ? 0.f : exp2f(m_run - m_new);
                l_run *= alpha;
                m_run = m_new;
                if (n >= 1) {                                        // O holds the tiles before this one: P V of tile n - 1 must have landed
                    if (!wait(PB_PFREE0 + ((n - 1) & 1), (uint32_t)((n - 1) >> 1))) { ok = false; break; }
                    tc_fence_after_sync();
#pragma unroll 1
                    for (int c0 = 0; c0 < 256; c0 += 32) {
                        uint32_t o[32];
                        tmem_ld32(tl + PFM_O + c0, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st32(tl + PFM_O + c0, o);
                    }
                    tmem_wait_st();
                }
            }
            // p = 2^(s sc - m) (a masked score gives 0) as bf16 hi + lo, written over the scores group by group: the 32 score
            // columns of keys 32 g .. 32 g + 31 become 16 columns of hi pairs and 16 columns of lo pairs
            const float nm = (m_run == -INFINITY) ? 0.f : -m_run;
#pragma unroll
            for (int g = 0; g < 4; g++) {
                uint32_t ph[16], pl[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float p0, p1;
                    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p0) : "f"(fmaf(sv[32 * g + i], sc, nm)));
                    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p1) : "f"(fmaf(sv[32 * g + i + 1], sc, nm)));
                    l_run += p0 + p1;
                    ph[i >> 1] = pack_bf16x2(p0, p1);
                    pl[i >> 1] = pack_bf16x2(p0 - __uint_as_float(ph[i >> 1] << 16), p1 - __uint_as_float(ph[i >> 1] & 0xffff0000u));
                }
                tmem_st16(sp + 32 * g, ph);
                tmem_st16(sp + 32 * g + 16, pl);
            }
            if (warp == 0) GDN_TSTAMP(n * 8 + 4);
            tmem_wait_st();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(PB_PREADY0 + (n & 1)));
            if (warp == 0) GDN_TSTAMP(n * 8 + 5);
        }
        // ---- epilogue: o = O / l; a split block first leaves (O, m, l) in the workspace, and the half that arrives last merges ----
        if (ok) ok = wait(PB_ODONE, 0);
        tc_fence_after_sync();
        const bool row_ok = ok && tok < a.S;
        __nv_bfloat16* orow = a.out + ((size_t)tok * ATT_H + kvh * ATT_GQA + (row & 3)) * ATT_D;
        float w_own = 1.f, w_other = 0.f;
        const float* other = nullptr;
        bool write_out = true;
        if (nparts == 2) {
            // The partial travels as one bulk copy each way: the rings are idle now (every tile has been consumed), so the rows are
            // staged there -- a thread's row is 1 KiB, written row by row the global stores would be 32 scattered segments per
            // instruction -- and the half that arrives last fetches the other half's image the same way.
            float* stage_f = reinterpret_cast<float*>(smem + PF_Q_BYTES);
            float* mine_s = stage_f + (size_t)row * (ATT_D + 4);
            float* mine_g = reinterpret_cast<float*>(a.ws + ws_parts_off16) + ((size_t)unit * 2 + part) * PF_PART_FLOATS;
            const float* other_g = reinterpret_cast<const float*>(a.ws + ws_parts_off16) + ((size_t)unit * 2 + (part ^ 1)) * PF_PART_FLOATS;
#pragma unroll 1
            for (int c0 = 0; c0 < 256; c0 += 32) {
                uint32_t o[32];
                tmem_ld32(tl + PFM_O + c0, o);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; i += 4)
                    *reinterpret_cast<float4*>(mine_s + c0 + i) = make_float4(__uint_as_float(o[i]), __uint_as_float(o[i + 1]), __uint_as_float(o[i + 2]), __uint_as_float(o[i + 3]));
            }
            *reinterpret_cast<float2*>(mine_s + ATT_D) = make_float2(m_run, l_run);
            fence_proxy_async_smem();
            asm volatile("bar.sync 1, 128;" ::: "memory");           // the four softmax warps
            if (tid == 0) {
                asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                             ::"l"(mine_g), "r"(smem_addr(stage_f)), "r"((uint32_t)(PF_PART_FLOATS * 4)) : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");      // the image is written (not merely read out of shared memory)
                __threadfence();
                s_last = (!aborted() && arrive(1 + unit) == 1u) ? 1 : 0;
                if (s_last) {
                    __threadfence();
                    asm volatile("fence.proxy.async;" ::: "memory");
                    mbar_expect_tx(bar(PB_QFULL), (uint32_t)(PF_PART_FLOATS * 4));      // (second use of this barrier: phase 1)
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                 ::"r"(smem_addr(stage_f)), "l"(other_g), "r"((uint32_t)(PF_PART_FLOATS * 4)), "r"(bar(PB_QFULL)) : "memory");
                }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            write_out = s_last != 0;
            if (write_out) {
                if (!wait(PB_QFULL, 1)) write_out = false;
                other = mine_s;                                      // the other half's row now sits where this thread's did
                const float2 ml = *reinterpret_cast<const float2*>(other + ATT_D);
                const float m = fmaxf(m_run, ml.x);
                w_own = m_run == -INFINITY ? 0.f : exp2f(m_run - m);
                w_other = ml.x == -INFINITY ? 0.f : exp2f(ml.x - m);
                // (sums in the order half 0, half 1 whichever half merges: the result does not depend on who arrived last)
                l_run = part == 0 ? fmaf(w_other, ml.y, w_own * l_run) : fmaf(w_own, l_run, w_other * ml.y);
            }
        }
        const float inv = l_run == 0.f ? 1.f : 1.f / l_run;
#pragma unroll 1
        for (int c0 = 0; c0 < 256; c0 += 32) {
            uint32_t o[32];
            tmem_ld32(tl + PFM_O + c0, o);
            tmem_wait_ld();
            if (row_ok && write_out) {
                float f[32];
                if (other) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        const float4 x = *reinterpret_cast<const float4*>(other + c0 + i);
                        const float xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const float own = __uint_as_float(o[i + e]);
                            f[i + e] = part == 0 ? fmaf(w_other, xs[e], own * w_own) : fmaf(w_own, own, xs[e] * w_other);
                        }
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i++) f[i] = __uint_as_float(o[i]);
                }
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    uint4 v;
                    v.x = pack_bf16x2(f[i] * inv, f[i + 1] * inv);
                    v.y = pack_bf16x2(f[i + 2] * inv, f[i + 3] * inv);
                    v.z = pack_bf16x2(f[i + 4] * inv, f[i + 5] * inv);
                    v.w = pack_bf16x2(f[i + 6] * inv, f[i + 7] * inv);
                    *reinterpret_cast<uint4*>(orow + c0 + i) = v;
                }
            }
        }
        tc_fence_before_sync();
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 4) tmem_dealloc(tb, 512);
    // the last block to get here -- blocks that gave up on a wait come here too -- starts the next call's epoch
    if (tid == 0 && n_split_units > 0) {
        __threadfence();
        if (arrive(0) == gridDim.x - 1) { *reinterpret_cast<volatile uint32_t*>(a.ws) = epoch + 1u; __threadfence(); }
    }
}

typedef CUresult (*PfEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                    const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// bf16 tensor (256, n1, n2) with strides s1 <= s2 (in elements) of the two outer dimensions; box = 64 x b1 x b2, 128-byte swizzle;
// rows outside the tensor read as zero
static bool make_map3(CUtensorMap* m, const void* base, long long n1, long long n2, long long s1, long long s2, int b1, int b2) {
    static PfEncodeTiledFn fn = nullptr;
    if (!fn) {
        cudaDriverEntryPointQueryResult qr;
        void* p = nullptr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) != cudaSuccess || qr != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            return false;
        }
        fn = reinterpret_cast<PfEncodeTiledFn>(p);
    }
    const cuuint64_t dims[3] = {(cuuint64_t)ATT_D, (cuuint64_t)n1, (cuuint64_t)n2};
    const cuuint64_t strides[2] = {(cuuint64_t)s1 * 2, (cuuint64_t)s2 * 2};
    const cuuint32_t box[3] = {64, (cuuint32_t)b1, (cuuint32_t)b2}, es[3] = {1, 1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// bytes of workspace with which launch_gqa_prefill may split the heaviest query blocks (0: the shape is never split)
static int pf_heavy_threshold(int S, int pos) {
    const int n_qb = (S + PF_QTOK - 1) / PF_QTOK;
    const int t_max = pf_tiles_of(n_qb - 1, S, pos);
    // splitting pays while there is at most one block per SM (the launch then lasts as long as the last query block), and only for
    // key ranges long enough to outweigh the merge (measured: S = 1024 and 2048 gain 12-13%, S = 512 and S = 4096 lose)
    if (2 * n_qb > 148 || t_max < 6) return 0;
    return max(2, (t_max + 1) / 2);
}
size_t gqa_prefill_workspace_bytes(int S, int pos) {
    if (S <= 0) return 0;
    const int th = pf_heavy_threshold(S, pos);
    if (th == 0) return 0;
    const int n_qb = (S + PF_QTOK - 1) / PF_QTOK;
    int n_heavy = 0;
    for (int qb = 0; qb < n_qb; qb++) n_heavy += pf_tiles_of(qb, S, pos) >= th ? 1 : 0;
    const size_t units = 2 * (size_t)n_heavy;
    return 16 + ((PF_WS_HEADER + 8 * (1 + units) + 15) & ~(size_t)15) + units * 2 * PF_PART_FLOATS * sizeof(float);
}

int launch_gqa_prefill(const void* q, const void* k, const void* v, void* out, int S, int pos, long long k_tok_stride, long long k_head_stride,
                       long long v_tok_stride, long long v_head_stride, void* workspace, size_t workspace_bytes, int* status, cudaStream_t stream) {
    if (S <= 0) return GDN_OK;
    CUtensorMap tq, tk, tv;
    memset(&tq, 0, sizeof(tq)); memset(&tk, 0, sizeof(tk)); memset(&tv, 0, sizeof(tv));
    const long long T = (long long)pos + S;
    const bool head_major = k_head_stride > k_tok_stride;            // [2, T, 256] rather than [T, 2, 256]
    if ((v_head_stride > v_tok_stride) != head_major) {
        set_error("gqa_prefill_attn: K and V must use the same layout");
        return GDN_E_SHAPE;
    }
    bool okm = make_map3(&tq, q, ATT_H, S, ATT_D, (long long)ATT_H * ATT_D, ATT_GQA, PF_QTOK);
    if (head_major) okm = okm && make_map3(&tk, k, T, ATT_KV, k_tok_stride, k_head_stride, PF_TK, 1) && make_map3(&tv, v, T, ATT_KV, v_tok_stride, v_head_stride, 32, 1);
    else okm = okm && make_map3(&tk, k, ATT_KV, T, k_head_stride, k_tok_stride, 1, PF_TK) && make_map3(&tv, v, ATT_KV, T, v_head_stride, v_tok_stride, 1, 32);
    if (!okm) {
        set_error("gqa_prefill_attn: cuTensorMapEncodeTiled failed (strides must be multiples of 8 elements)");
        return GDN_E_UNSUPPORTED;
    }
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        if (cudaFuncSetAttribute(gqa_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM) != cudaSuccess)
            return check_launch("gqa_prefill smem attribute");
        attr_set[dev] = true;
    }
    PrefillAttnArgs a;
    a.out = static_cast<__nv_bfloat16*>(out); a.S = S; a.pos = pos; a.status = status; a.kv_head_major = head_major ? 1 : 0;
    const int n_qb = (S + PF_QTOK - 1) / PF_QTOK;
    // with a workspace the query blocks with the most keys are split in two along the keys (the causal triangle is otherwise as slow
    // as its last block whenever there are not several blocks per SM)
    a.heavy_tiles = 0;
    a.ws = nullptr;
    int n_heavy = 0;
    const size_t need = gqa_prefill_workspace_bytes(S, pos);
    if (workspace && need > 0 && workspace_bytes >= need) {
        a.heavy_tiles = pf_heavy_threshold(S, pos);
        a.ws = static_cast<unsigned char*>(workspace);
        for (int qb = 0; qb < n_qb; qb++) n_heavy += pf_tiles_of(qb, S, pos) >= a.heavy_tiles ? 1 : 0;
    }
    gqa_prefill_tc_kernel<<<(n_qb + n_heavy) * ATT_KV, PF_THREADS, PF_SMEM, stream>>>(a, tq, tk, tv);
    return check_launch("gqa_prefill_attn");
}

}  // namespace gdn

#ifdef GDN_TIMING
extern "C" __attribute__((visibility("default"))) int gdn_timing_log_d(long long* out_host, int n) {
    return cudaMemcpyFromSymbol(out_host, gdn::g_tlog, sizeof(long long) * n) == cudaSuccess ? 0 : -5;
}
#endif
