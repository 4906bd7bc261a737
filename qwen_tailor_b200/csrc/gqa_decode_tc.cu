// GQA decode attention, head_dim 256, on the Blackwell tensor cores (tcgen05 / TMEM / TMA) -- the path for paged caches whose
// pages hold a multiple of 64 keys (a 64-key tile then lies inside one page and is fetched by tensor-map copies).
//
// Same contract as gqa_decode.cu (the reference's `attn_b`, qwen35/batch.py:141-237): for row r = b*M + j, softmax(q K^T / 16) V over
// the keys [0, ctx_len[b] + j], the M rows of the call taken from the call's inputs and appended to the cache.  Same balanced
// split-KV plan, partial format and merge.  What differs is the arithmetic engine: warp-level MMAs (mma.sync) run at about a
// fifteenth of the tcgen05 rate on this part and left that kernel bound by its MMA count, far below the memory roofline.
//
// Per 64-key tile, with the 16 query rows (4 q-heads of the KV head x M <= 4 rows) as rows 0..15 of an M = 128 product:
//     S [128 x 64]   = Q K^T        16 MMAs (K = 256 dims), A = Q from shared memory, B = the K tile as TMA wrote it
//     P              = 2^(S sc - m) on 16 threads (one query row each), bf16 hi + lo pairs into tensor memory
//     O [128 x 256] += P V          8 MMAs (K = 64 keys, hi and lo), A = P from tensor memory, B = the V tile read N-major
// Rows 16..127 of the Q operand view whatever follows Q in shared memory; their products land in accumulator lanes that nobody
// reads.  S and P are double buffered in tensor memory (O 256 + 2 x 64 + 2 x 64 columns = 512), so the softmax of tile t runs
// while the tensor pipe forms the scores of tile t + 1.  The running maximum is only raised when a tile exceeds it by more than
// 2^8 (P then stays below 256, far inside bf16 / fp32 range), which makes the rescale of O -- a round trip through registers --
// rare; the final result is exact either way because l and O carry the same reference.
//
// Roles (128 threads, one persistent block per SM): warp 0 softmax / epilogue (lanes 0..15 own the query rows), warp 1 lane 0
// issues the MMAs, warp 2 is the TMA producer (three-stage ring of K + V tiles), warp 3 stages Q and appends the new rows.
// Every wait is bounded; a wait that gives up sets the device status word and the block runs out its loops without touching
// the tensor cores again.
#include <cstring>
#include "gqa_common.cuh"
#include "sm100_prims.cuh"

namespace gdn {

using namespace sm100;

constexpr uint32_t TCM_O = 0, TCM_S0 = 256, TCM_P0 = 384;            // O [256], S buffers [64] x 2, P buffers [hi 32 | lo 32] x 2
enum { TB_FULL0 = 0, TB_EMPTY0 = 3, TB_SDONE0 = 6, TB_SFREE0 = 8, TB_PREADY0 = 10, TB_PFREE0 = 12, TB_ODONE = 14, TB_COUNT = 15 };
constexpr float TC_RESCALE_STEP = 8.f;                               // log2 units

__global__ void __launch_bounds__(TC_THREADS, 1)
gqa_decode_tc_kernel(const AttnArgs a, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV) {
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ uint64_t bars[TB_COUNT];
    __shared__ uint32_t tmem_slot;
    __shared__ int s_abort, s_last;
    __shared__ float s_w[(148 + 2) * 16];                            // merge weights: [partials of a pair][16 rows], then 1 / sum

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int M = a.M, P = a.P;
    const int* cum = meta_cum(a.meta);
    const long long N = a.meta[0];
    const int G = a.meta[1];                                         // working blocks = min(grid, tiles)
    if ((int)blockIdx.x >= G) return;
    long long lo = (long long)blockIdx.x * N / G;
    const long long hi = (long long)(blockIdx.x + 1) * N / G;
    if (lo >= hi) return;
    const uint32_t sbase = smem_addr(smem);
    if (sbase & 1023u) { if (tid == 0) atomicExch(a.status, 4); return; }
    auto bar = [&](int i) -> uint32_t { return smem_addr(&bars[i]); };
    if (tid == 0) {
        for (int i = 0; i < 3; i++) { mbar_init(bar(TB_FULL0 + i), 1); mbar_init(bar(TB_EMPTY0 + i), 1); }
        for (int i = 0; i < 2; i++) { mbar_init(bar(TB_SDONE0 + i), 1); mbar_init(bar(TB_SFREE0 + i), 1); mbar_init(bar(TB_PREADY0 + i), 1); mbar_init(bar(TB_PFREE0 + i), 1); }
        mbar_init(bar(TB_ODONE), 1);
        s_abort = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
    }
    if (warp == 1) { tmem_alloc(smem_addr(&tmem_slot), 512); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tb = tmem_slot;
    GDN_BSTAMP(0);

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

    const uint32_t sQ = sbase, sKV = sbase + TC_Q_BYTES;
    uint32_t n0 = 0;                                                 // tiles this block has put through the ring before the current pair
    uint32_t pairs_done = 0;
    int pair;                                                        // pair that owns tile lo: cum[pair] <= lo < cum[pair + 1]
    {
        int l = 0, r = P - 1;
        while (l < r) { const int m = (l + r + 1) >> 1; if (cum[m] <= lo) l = m; else r = m - 1; }
        pair = l;
    }
    for (; lo < hi; pair++) {
        if (cum[pair + 1] <= lo) continue;                           // pairs without tiles (rejected sequences)
        const long long seg_end = min(hi, (long long)cum[pair + 1]);
        const int ta = (int)(lo - cum[pair]), tbk = (int)(seg_end - cum[pair]);      // this block's tiles of the pair: [ta, tbk)
        const int slot = meta_base(a.meta, P)[pair] + ((int)blockIdx.x - meta_first(a.meta, P)[pair]);
        lo = seg_end;
        const int b = pair / ATT_KV, kvh = pair % ATT_KV;
        const int ctx = a.ctx_len[b];
        const int all_ctx_tiles = (ctx + TK - 1) / TK;               // tile index all_ctx_tiles holds the rows of this call
        const int ctx_tiles = max(0, min(tbk, all_ctx_tiles) - ta);
        const int ntiles = tbk - ta;
        const int k_begin = ta * TK;
        const int k_end = min(ctx, (ta + ctx_tiles) * TK);
        const int* table = a.block_table + (size_t)b * a.max_pages;

        // ---- prologue: Q rows into the operand slabs (row r = j*4 + hq <-> q[(b*M + j), kvh*4 + hq, :]; rows >= 4M zero) and, in the
        //      block that owns the pair's first tile, the new rows into the cache (readers take them from the inputs) ----
        if (warp == 3) {
            for (int i = lane; i < 16 * 32; i += 32) {
                const int r = i >> 5, c = i & 31, j = r >> 2, hq = r & 3;
                uint4 v = make_uint4(0, 0, 0, 0);
                if (j < M) v = reinterpret_cast<const uint4*>(a.q + (((size_t)b * M + j) * ATT_H + kvh * ATT_GQA + hq) * ATT_D)[c];
                unsigned char* dst = smem + (c >> 3) * 4096 + r * 128 + (((c & 7) ^ (r & 7)) << 4);
                *reinterpret_cast<uint4*>(dst) = v;
                *reinterpret_cast<uint4*>(dst + 2048) = v;             // rows 16..31 repeat rows 0..15 (r + 16 has the same r & 7)
            }
            fence_proxy_async_smem();
            if (ta == 0) {
                for (int i = lane; i < M * 64; i += 32) {
                    const int jj = i >> 6, c = i & 31, isv = (i >> 5) & 1;
                    const int pos = ctx + jj;
                    const int page = table[pos / a.page_size];
                    if (page < 0 || page >= a.n_pages) { atomicExch(a.status, 1); continue; }
                    const __nv_bfloat16* src = (isv ? a.v_new : a.k_new) + (((size_t)b * M + jj) * ATT_KV + kvh) * ATT_D;
                    __nv_bfloat16* dst = (isv ? a.v_pages : a.k_pages) + (((size_t)page * ATT_KV + kvh) * a.page_size + pos % a.page_size) * ATT_D;
                    reinterpret_cast<uint4*>(dst)[c] = reinterpret_cast<const uint4*>(src)[c];
                }
            }
        }
        __syncthreads();

        if (warp == 2) {
            // ================= producer: keep the ring full with the tiles [ta, tbk) of this pair =================
            for (int t = 0; t < ntiles && !aborted(); t++) {
                const uint32_t n = n0 + t;
                const int stage = n % ATT_STAGES;
                if (n >= (uint32_t)ATT_STAGES && !wait(TB_EMPTY0 + stage, (n / ATT_STAGES) - 1)) break;
                const uint32_t dK = sKV + stage * 2 * TILE_BYTES, dV = dK + TILE_BYTES;
                if (t < ctx_tiles) {
                    if (lane == 0) {
                        const int key = k_begin + t * TK;
                        int page = table[key / a.page_size];
                        if (page < 0 || page >= a.n_pages) { atomicExch(a.status, 1); page = 0; }      // reported; page 0 is read in its place
                        const int row = key % a.page_size;
                        mbar_expect_tx(bar(TB_FULL0 + stage), 2 * TILE_BYTES);
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                                         ::"r"(dK + j * 8192), "l"(&tmK), "r"(bar(TB_FULL0 + stage)), "r"(64 * j), "r"(row), "r"(kvh), "r"(page) : "memory");
                            asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                                         ::"r"(dV + j * 8192), "l"(&tmV), "r"(bar(TB_FULL0 + stage)), "r"(64 * j), "r"(row), "r"(kvh), "r"(page) : "memory");
                        }
                    }
                } else {
                    // the rows of this call, copied from k_new / v_new; rows M..15 are zeroed (the P V product of this tile reads 16 keys)
                    for (int i = lane; i < 16 * 32; i += 32) {
                        const int r = i >> 5, c = i & 31;
                        uint4 kv4 = make_uint4(0, 0, 0, 0), vv4 = make_uint4(0, 0, 0, 0);
                        if (r < M) {
                            const size_t off = (((size_t)b * M + r) * ATT_KV + kvh) * ATT_D;
                            kv4 = reinterpret_cast<const uint4*>(a.k_new + off)[c];
                            vv4 = reinterpret_cast<const uint4*>(a.v_new + off)[c];
                        }
                        *reinterpret_cast<uint4*>(smem + TC_Q_BYTES + stage * 2 * TILE_BYTES + swz_t(r, c)) = kv4;
                        *reinterpret_cast<uint4*>(smem + TC_Q_BYTES + stage * 2 * TILE_BYTES + TILE_BYTES + swz_t(r, c)) = vv4;
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar(TB_FULL0 + stage));
                }
            }
        } else if (warp == 1) {
            // ================= MMA issuer =================
            if (lane == 0) {
                constexpr uint32_t I_QK = idesc_bf16(128, 64, 0, 0);
                constexpr uint32_t I_PV = idesc_bf16(128, 256, 0, 1);    // B = V read N-major (dims contiguous)
                constexpr uint32_t HI_K = smem_desc_hi_sw128(1024);
                auto issue_pv = [&](uint32_t m, bool first, bool new_tile) -> bool {
                    const int buf = m & 1, stage = m % ATT_STAGES;
                    if (!wait(TB_PREADY0 + buf, m >> 1)) return false;
                    tc_fence_after_sync();
                    GDN_TSTAMP(m * 8 + 2);
                    const uint32_t vlo = smem_desc_lo(sKV + stage * 2 * TILE_BYTES + TILE_BYTES, 8192);
                    const int nks = new_tile ? 1 : 4;                    // the tile of this call's own rows holds at most 16 keys
                    for (int part = 0; part < 2; part++)
                        for (int ks = 0; ks < nks; ks++) {
                            const uint32_t acol = tb + TCM_P0 + buf * 64 + part * 32 + ks * 8;
                            if (first && part == 0 && ks == 0) mma_ts_w<false>(tb + TCM_O, acol, vlo + ks * 128, HI_K, I_PV);
                            else mma_ts_w<true>(tb + TCM_O, acol, vlo + ks * 128, HI_K, I_PV);
                        }
                    mma_commit(bar(TB_EMPTY0 + stage));
                    mma_commit(bar(TB_PFREE0 + buf));
                    GDN_TSTAMP(m * 8 + 3);
                    return true;
                };
                bool ok = true;
                for (int t = 0; t < ntiles && ok && !aborted(); t++) {
                    const uint32_t n = n0 + t;
                    const int buf = n & 1, stage = n % ATT_STAGES;
                    ok = wait(TB_FULL0 + stage, n / ATT_STAGES) && (n < 2 || wait(TB_SFREE0 + buf, (n >> 1) - 1));
                    if (!ok) break;
                    tc_fence_after_sync();
                    GDN_TSTAMP(n * 8 + 0);
                    const uint32_t klo = smem_desc_lo(sKV + stage * 2 * TILE_BYTES, 16), qlo = smem_desc_lo(sQ, 16);
#pragma unroll
                    for (int ks = 0; ks < 16; ks++) {
                        const uint32_t qo = (ks >> 2) * (4096 >> 4) + (ks & 3) * 2, ko = (ks >> 2) * (8192 >> 4) + (ks & 3) * 2;
                        if (ks == 0) mma_ss_w<false>(tb + TCM_S0 + buf * 64, qlo + qo, HI_K, klo + ko, HI_K, I_QK);
                        else mma_ss_w<true>(tb + TCM_S0 + buf * 64, qlo + qo, HI_K, klo + ko, HI_K, I_QK);
                    }
                    mma_commit(bar(TB_SDONE0 + buf));
                    GDN_TSTAMP(n * 8 + 1);
                    if (t >= 1) ok = issue_pv(n - 1, t == 1, (t - 1) >= ctx_tiles);
                }
                if (ok && !aborted()) ok = issue_pv(n0 + ntiles - 1, ntiles == 1, (ntiles - 1) >= ctx_tiles);
                if (ok) mma_commit(bar(TB_ODONE));
            }
        } else if (warp == 0) {
            // ================= softmax: lanes r and r + 16 share query row r, 32 keys of every tile each =================
            const float sc = 0.0625f * 1.4426950408889634f;          // 256^-1/2 (qwen35/batch.py:176), scores kept in log2 units
            float m_run = -INFINITY, l_run = 0.f;                    // m: the row's reference (same in both lanes); l: this lane's share
            const int row = lane & 15, half = lane >> 4;
            const int my_j = row >> 2;                               // chained row of this query row
            const bool real = row < 4 * M;                           // rows beyond the query rows are zero padding: everything masked
            bool ok = true;
            for (int t = 0; t < ntiles && ok; t++) {
                const uint32_t n = n0 + t;
                const int buf = n & 1, stage = n % ATT_STAGES;
                const bool new_tile = t >= ctx_tiles;
                const int limit = new_tile ? M : k_end - (k_begin + t * TK);     // keys of the tile that exist
                if (!wait(TB_SDONE0 + buf, n >> 1)) { ok = false; break; }
                tc_fence_after_sync();
                GDN_TSTAMP(n * 8 + 4);
                float s[32];
                {
                    uint32_t r0[32], r1[32];
                    tmem_ld32(tb + TCM_S0 + buf * 64, r0);
                    tmem_ld32(tb + TCM_S0 + buf * 64 + 32, r1);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i++) s[i] = __uint_as_float(half ? r1[i] : r0[i]);
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(TB_SFREE0 + buf));    // the score columns may take tile n + 2
                GDN_TSTAMP(n * 8 + 5);
                float mt = -INFINITY;
                if (!real || new_tile || limit < TK) {               // masks only where a tile is not full
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        const int k = half * 32 + i;
                        const bool vis = real && (new_tile ? (k < M && k <= my_j) : (k < limit));
                        s[i] = vis ? s[i] : -INFINITY;
                    }
                }
#pragma unroll
                for (int i = 0; i < 32; i++) mt = fmaxf(mt, s[i]);
                mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 16)) * sc;       // (sc > 0: the maximum of the scaled scores)
                // raise the reference only when it is far behind (or not set yet); O is rescaled then -- all lanes take part in the
                // tensor-memory round trip, each with its own factor
                const bool raise = mt > m_run + TC_RESCALE_STEP || (m_run == -INFINITY && mt != -INFINITY);
                if (__any_sync(0xffffffffu, raise)) {
                    const float m_new = raise ? mt : m_run;
                    const float alpha = (m_run == -INFINITY) ? 0.f : exp2f(m_run - m_new);
                    l_run *= alpha;
                    m_run = m_new;
                    if (t >= 1) {                                    // O holds the tiles before this one: P V of tile n - 1 must have landed
                        if (!wait(TB_PFREE0 + ((n - 1) & 1), (n - 1) >> 1)) { ok = false; break; }
                        tc_fence_after_sync();
#pragma unroll 1
                        for (int c0 = 0; c0 < 256; c0 += 32) {
                            uint32_t o[32];
                            tmem_ld32(tb + TCM_O + c0, o);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                            tmem_st32(tb + TCM_O + c0, o);
                        }
                        tmem_wait_st();
                    }
                }
                // p = 2^(s sc - m); a masked score (-inf) gives 0, and a row without any visible key so far keeps m = -inf: p = 0 there
                uint32_t mh[16], ml[16];
                const float nm = (m_run == -INFINITY) ? 0.f : -m_run;
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float p0, p1;
                    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p0) : "f"(fmaf(s[i], sc, nm)));
                    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p1) : "f"(fmaf(s[i + 1], sc, nm)));
                    l_run += p0 + p1;
                    mh[i >> 1] = pack_bf16x2(p0, p1);
                    ml[i >> 1] = pack_bf16x2(p0 - __uint_as_float(mh[i >> 1] << 16), p1 - __uint_as_float(mh[i >> 1] & 0xffff0000u));
                }
                // this lane's 32 keys are one half of the row's P columns; the other half of ITS accumulator row is zero
                uint32_t ph[32], pl[32];
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    ph[i] = half ? 0u : mh[i]; ph[16 + i] = half ? mh[i] : 0u;
                    pl[i] = half ? 0u : ml[i]; pl[16 + i] = half ? ml[i] : 0u;
                }
                // value rows past the end of the context hold whatever the page holds there and must not reach the MMA (0 x NaN)
                if (!new_tile && limit < TK) {
                    if (!wait(TB_FULL0 + stage, n / ATT_STAGES)) { ok = false; break; }      // (long complete: orders these writes after the copy's)
                    for (int i = lane; i < (TK - limit) * 32; i += 32)
                        *reinterpret_cast<uint4*>(smem + TC_Q_BYTES + stage * 2 * TILE_BYTES + TILE_BYTES + swz_t(limit + (i >> 5), i & 31)) = make_uint4(0, 0, 0, 0);
                    fence_proxy_async_smem();
                }
                GDN_TSTAMP(n * 8 + 6);
                if (n >= 2 && !wait(TB_PFREE0 + buf, (n >> 1) - 1)) { ok = false; break; }      // P V of tile n - 2 has read this buffer
                tc_fence_after_sync();
                tmem_st32(tb + TCM_P0 + buf * 64, ph);
                tmem_st32(tb + TCM_P0 + buf * 64 + 32, pl);
                tmem_wait_st();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(TB_PREADY0 + buf));
                GDN_TSTAMP(n * 8 + 7);
            }
            // ---- epilogue: O / l (the whole pair was this block's) or a partial (max, sum, O) for the merge ----
            if (ok) ok = wait(TB_ODONE, pairs_done);
            tc_fence_after_sync();
            const int nsp = meta_base(a.meta, P)[pair + 1] - meta_base(a.meta, P)[pair];
            float* part = a.part + (size_t)slot * PART_STRIDE;
            l_run += __shfl_xor_sync(0xffffffffu, l_run, 16);
            const bool row_ok = ok && lane < 4 * M;                  // lanes 0..15 write the rows
            const float inv = l_run == 0.f ? 1.f : 1.f / l_run;      // sum == 0 guard as qwen35/batch.py:216
            __nv_bfloat16* orow = a.out + (((size_t)b * M + (row >> 2)) * ATT_H + kvh * ATT_GQA + (row & 3)) * ATT_D;
#pragma unroll 1
            for (int c0 = 0; c0 < 256; c0 += 32) {
                uint32_t o[32];
                tmem_ld32(tb + TCM_O + c0, o);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) + __shfl_xor_sync(0xffffffffu, __uint_as_float(o[i]), 16));
                if (row_ok) {
                    if (nsp == 1) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            uint4 v;
                            v.x = pack_bf16x2(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
                            v.y = pack_bf16x2(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
                            v.z = pack_bf16x2(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
                            v.w = pack_bf16x2(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
                            *reinterpret_cast<uint4*>(orow + c0 + i) = v;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            *reinterpret_cast<float4*>(part + lane * ATT_D + c0 + i) =
                                make_float4(__uint_as_float(o[i]), __uint_as_float(o[i + 1]), __uint_as_float(o[i + 2]), __uint_as_float(o[i + 3]));
                    }
                }
            }
            if (row_ok && nsp > 1) { part[16 * ATT_D + 2 * lane] = m_run; part[16 * ATT_D + 2 * lane + 1] = l_run; }
            tc_fence_before_sync();
        }
        n0 += ntiles;
        pairs_done++;
        GDN_BSTAMP(1 + 2 * (pairs_done > 1));

        // ---- merge: the block that writes the last partial of a pair combines them (the counters were zeroed by this call's plan kernel) ----
        const int* pbase = meta_base(a.meta, P);
        const int nsp = pbase[pair + 1] - pbase[pair];
        __threadfence();
        __syncthreads();
        if (nsp > 1) {
            if (tid == 0) s_last = (!aborted() && atomicAdd(meta_count(a.meta, P) + pair, 1) == nsp - 1) ? 1 : 0;
            __syncthreads();
            if (s_last && nsp <= 148) {
                __threadfence();
                const float* pb = a.part + (size_t)pbase[pair] * PART_STRIDE;
                for (int i = tid; i < nsp * 16; i += TC_THREADS) s_w[i] = __ldcg(pb + (size_t)(i >> 4) * PART_STRIDE + 16 * ATT_D + 2 * (i & 15));
                __syncthreads();
                if (tid < 16) {
                    float ms = -INFINITY, lsum = 0.f;
                    for (int sp = 0; sp < nsp; sp++) ms = fmaxf(ms, s_w[sp * 16 + tid]);
                    for (int sp = 0; sp < nsp; sp++) {
                        const float m = s_w[sp * 16 + tid];
                        const float w = (m == -INFINITY) ? 0.f : exp2f(m - ms);
                        lsum += w * __ldcg(pb + (size_t)sp * PART_STRIDE + 16 * ATT_D + 2 * tid + 1);
                        s_w[sp * 16 + tid] = w;
                    }
                    s_w[nsp * 16 + tid] = lsum == 0.f ? 1.f : 1.f / lsum;
                }
                __syncthreads();
                __nv_bfloat16* out_pair = a.out + ((size_t)b * M * ATT_H + kvh * ATT_GQA) * ATT_D;
                // thread = (row pair, 16 dims): every partial contributes 8 independent 16-byte loads, and the loop over partials is
                // unrolled, so a few dozen loads are in flight per thread (the partials sit in L2; the merge is latency-bound)
                const int rp = tid >> 4, d0 = (tid & 15) * 16;
                float acc[2][16];
#pragma unroll
                for (int q = 0; q < 2; q++)
#pragma unroll
                    for (int i = 0; i < 16; i++) acc[q][i] = 0.f;
#pragma unroll 4
                for (int sp = 0; sp < nsp; sp++) {
#pragma unroll
                    for (int q = 0; q < 2; q++) {
                        const int r = 2 * rp + q;
                        const float w = s_w[sp * 16 + r];
                        const float4* pp = reinterpret_cast<const float4*>(pb + (size_t)sp * PART_STRIDE + r * ATT_D + d0);
#pragma unroll
                        for (int v4 = 0; v4 < 4; v4++) {
                            const float4 x = __ldcg(pp + v4);
                            acc[q][4 * v4] += w * x.x; acc[q][4 * v4 + 1] += w * x.y; acc[q][4 * v4 + 2] += w * x.z; acc[q][4 * v4 + 3] += w * x.w;
                        }
                    }
                }
#pragma unroll
                for (int q = 0; q < 2; q++) {
                    const int r = 2 * rp + q;
                    if (r < 4 * M) {
                        const float inv = s_w[nsp * 16 + r];
                        __nv_bfloat16* dst = out_pair + ((size_t)(r >> 2) * ATT_H + (r & 3)) * ATT_D + d0;
                        uint4 v0, v1;
                        v0.x = pack_bf16x2(acc[q][0] * inv, acc[q][1] * inv); v0.y = pack_bf16x2(acc[q][2] * inv, acc[q][3] * inv);
                        v0.z = pack_bf16x2(acc[q][4] * inv, acc[q][5] * inv); v0.w = pack_bf16x2(acc[q][6] * inv, acc[q][7] * inv);
                        v1.x = pack_bf16x2(acc[q][8] * inv, acc[q][9] * inv); v1.y = pack_bf16x2(acc[q][10] * inv, acc[q][11] * inv);
                        v1.z = pack_bf16x2(acc[q][12] * inv, acc[q][13] * inv); v1.w = pack_bf16x2(acc[q][14] * inv, acc[q][15] * inv);
                        reinterpret_cast<uint4*>(dst)[0] = v0;
                        reinterpret_cast<uint4*>(dst)[1] = v1;
                    }
                }
            }
            __syncthreads();                                         // s_w and s_last are reused by the block's next pair
        }
        GDN_BSTAMP(2 + 2 * (pairs_done > 1));
    }
    tc_fence_before_sync();
    __syncthreads();
    GDN_BSTAMP(5);
    if (warp == 1) tmem_dealloc(tb, 512);
}

int launch_gqa_decode_tc(const AttnArgs& a, const CUtensorMap& tk, const CUtensorMap& tv, cudaStream_t stream) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        if (cudaFuncSetAttribute(gqa_decode_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM) != cudaSuccess)
            return check_launch("gqa_decode_tc smem attribute");
        attr_set[dev] = true;
    }
    gqa_decode_tc_kernel<<<a.G, TC_THREADS, TC_SMEM, stream>>>(a, tk, tv);
    return check_launch("gqa_decode_tc");
}

}  // namespace gdn

#ifdef GDN_TIMING
extern "C" __attribute__((visibility("default"))) int gdn_timing_log_c(long long* out_host, int n) {
    return cudaMemcpyFromSymbol(out_host, gdn::g_tlog, sizeof(long long) * n) == cudaSuccess ? 0 : -5;
}
#endif
