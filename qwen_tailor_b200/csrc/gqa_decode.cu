// GQA decode attention, head_dim 256, 8 query heads / 2 KV heads, over a paged bf16 KV cache.
//
// Replaces the reference's `attn_b` Metal kernel (qwen35/batch.py:141-237): for row r = b*M + j, softmax(q K^T / 16) V over
// the keys [0, ctx_len[b] + j]; the keys/values of the M rows of this call are taken from the call's inputs (never from the
// cache, so the in-place append needs no ordering against readers, batch.py:143-148,182) and are appended to the cache at
// positions ctx_len[b] + j.  The reference's contiguous slot pool [S+1, 2, Lmax, 256] is the special case
// page_size = Lmax, block_table[b] = {slot}.
//
// The kernel is bound by streaming K and V once (2 KiB per cached token and layer).  Design:
//   * balanced split-KV: the 64-key tiles of all (sequence, kv head) pairs form one list (a tiny plan kernel builds its prefix
//     sums from ctx_len on the device), and one persistent block per SM takes a contiguous 1/n-th of it, so a ragged batch
//     loads every SM equally whatever the context lengths are.  Where a block's range crosses from one pair to the next, or
//     ends inside one, it writes a partial (max, sum, O) to a caller-provided fp32 workspace; the block that writes the
//     last partial of a pair (an arrival counter tells it) merges them and stores the bf16 rows.  A pair that lies inside one
//     block's range is stored directly.
//   * GQA packing: the 4 query heads of a KV head times the M <= 4 chained rows form the 16 rows of a warp-level
//     m16n8k16 bf16 MMA, so each K/V byte is read once for up to 16 query rows (at M = 4 plain FMAs could not keep up with
//     HBM).  The 8 warps are 4 key groups x 2 halves of the head dim: a warp computes the scores of 8 of its group's 16 keys,
//     swaps them with its partner through shared memory (warp-level MMAs run at a fraction of the tcgen05 rate on this part and
//     the kernel is bound by their number, so nothing is computed twice), and does P.V for its 128 of the 256 dims with its own
//     online-softmax state.
//   * K/V tiles (64 keys x 512 B) are gathered page by page with 16-byte cp.async into XOR-swizzled shared memory, three
//     stages (192 KiB per SM, two tiles in flight while one is consumed).  The page lookup of a tile's 64 keys is done once
//     (one thread per key) and shared through shared memory.
//   * the probabilities are fed to the P.V MMA as a bf16 hi + lo pair, so the result carries fp32-level accuracy like the
//     reference's fp32 accumulation of exp_score * v.
#include <cuda.h>
#include <cstring>
#include "gqa_common.cuh"
#include "sm100_prims.cuh"

namespace gdn {

__global__ void __launch_bounds__(256) gqa_decode_plan_kernel(const AttnArgs a) {
    __shared__ int s_sum[256];
    const int tid = threadIdx.x, P = a.P;
    int* cum = meta_cum(a.meta);
    int* base = meta_base(a.meta, P);
    int* first = meta_first(a.meta, P);
    const int chunk = (P + 255) / 256, p0 = min(P, tid * chunk), p1 = min(P, p0 + chunk);
    auto tiles_of = [&](int p) -> int {
        const int ctx = a.ctx_len[p / ATT_KV];
        if (ctx < 0 || (long long)ctx + a.M > (long long)a.max_pages * a.page_size) { atomicExch(a.status, 1); return 0; }
        // cached keys + one tile for the rows of this call + the weight of the pair's epilogue: `tail_tiles` tiles without work,
        // so that a block that finishes a pair (reads out the accumulator, maybe merges) is given that much less to stream
        return (ctx + TK - 1) / TK + 1 + a.tail_tiles;
    };
    auto scan = [&](int local) -> int {                               // exclusive prefix of `local` over the block
        int x = local;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const int y = __shfl_up_sync(0xffffffffu, x, o); if ((tid & 31) >= o) x += y; }
        __syncthreads();
        if ((tid & 31) == 31) s_sum[tid >> 5] = x;
        __syncthreads();
        int before = 0;
        for (int w = 0; w < (tid >> 5); w++) before += s_sum[w];
        return before + x - local;
    };
    int local = 0;
    for (int p = p0; p < p1; p++) local += tiles_of(p);
    int run = scan(local);
    for (int p = p0; p < p1; p++) { cum[p] = run; run += tiles_of(p); }
    if (p1 == P && p0 <= P && tid == min(255, (P - 1) / max(chunk, 1))) { cum[P] = run; a.meta[0] = run; }
    __syncthreads();
    __threadfence_block();
    const long long N = cum[P];
    // with fewer tiles than blocks only the first N blocks work (one tile each): every working block then has a non-empty range,
    // so the blocks of a pair are consecutive and each of its partial slots is written
    const int G = (int)min((long long)a.G, max(N, 1ll));
    if (tid == 0) a.meta[1] = G;
    // a pair's partials come from the blocks that hold its tiles with work (the weight tiles at its end carry none)
    local = 0;
    for (int p = p0; p < p1; p++) {
        const int t = cum[p + 1] - cum[p];
        local += t > 0 ? block_of_tile(cum[p + 1] - 1 - a.tail_tiles, G, N) - block_of_tile(cum[p], G, N) + 1 : 0;
    }
    run = scan(local);
    for (int p = p0; p < p1; p++) {
        const int t = cum[p + 1] - cum[p];
        const int f = t > 0 ? block_of_tile(cum[p], G, N) : 0;
        first[p] = f;
        base[p] = run;
        run += t > 0 ? block_of_tile(cum[p + 1] - 1 - a.tail_tiles, G, N) - f + 1 : 0;
    }
    if (tid == min(255, (P - 1) / max(chunk, 1))) base[P] = run;
    int* count = meta_count(a.meta, P);
    for (int p = tid; p < P; p += 256) count[p] = 0;
}

// TMA = false: every warp gathers its share of a tile with 16-byte cp.async (any page size).
// TMA = true (pages hold a multiple of 64 keys, so a tile lies inside one page): a ninth warp is the producer -- one lane issues
// eight tensor-map copies per tile into a three-stage ring guarded by full / empty mbarriers, the eight math warps never issue
// or wait for copies and meet no block-wide barrier inside a pair.
template <bool TMA>
__global__ void __launch_bounds__(TMA ? ATT_THREADS + 32 : ATT_THREADS, 1)
gqa_decode_split_kernel(const AttnArgs a, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV) {
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ uint64_t ring_bar[2 * ATT_STAGES + 1];               // full[3], empty[3], pair finished (TMA path)
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int M = a.M, P = a.P;
    const int* cum = meta_cum(a.meta);
    const long long N = a.meta[0];
    const int G = a.meta[1];                                         // working blocks = min(grid, tiles)
    if ((int)blockIdx.x >= G) return;
    long long lo = (long long)blockIdx.x * N / G;
    const long long hi = (long long)(blockIdx.x + 1) * N / G;
    if (lo >= hi) return;
    const bool producer = TMA && warp == 8;
    auto csync = [&]() {                                             // barrier among the 256 math threads
        if (TMA) asm volatile("bar.sync 1, 256;" ::: "memory"); else __syncthreads();
    };
    auto rbar = [&](int i) -> uint32_t { return smem_u32(&ring_bar[i]); };
    uint32_t ring_n = 0;                                             // tiles this block has put through the ring so far (TMA path)
    uint32_t pairs_done = 0;
    if (TMA) {
        // the 128-byte-swizzled boxes start 16 * ROWB = 8 KiB into the dynamic shared memory: its base must be 1024-byte aligned
        if (smem_u32(smem) & 1023u) { if (tid == 0) atomicExch(a.status, 4); return; }
        if (tid == 0) {
            for (int i = 0; i < ATT_STAGES; i++) { sm100::mbar_init(rbar(i), 1); sm100::mbar_init(rbar(ATT_STAGES + i), 8); }
            sm100::mbar_init(rbar(2 * ATT_STAGES), 8);
            sm100::fence_barrier_init();
        }
        __syncthreads();
    }
    int pair;                                                        // pair that owns tile lo: cum[pair] <= lo < cum[pair + 1]
    {
        int l = 0, r = P - 1;
        while (l < r) { const int m = (l + r + 1) >> 1; if (cum[m] <= lo) l = m; else r = m - 1; }
        pair = l;
    }
  for (; lo < hi; pair++) {
    if (cum[pair + 1] <= lo) continue;                               // pairs without tiles (rejected sequences)
    const long long seg_end = min(hi, (long long)cum[pair + 1]);
    const int ta = (int)(lo - cum[pair]), tb = (int)(seg_end - cum[pair]);      // this block's tiles of the pair: [ta, tb)
    const int slot = meta_base(a.meta, P)[pair] + ((int)blockIdx.x - meta_first(a.meta, P)[pair]);
    lo = seg_end;
    const int b = pair / ATT_KV, kvh = pair % ATT_KV;
    const int ctx = a.ctx_len[b];
    const int all_ctx_tiles = (ctx + TK - 1) / TK;                   // tile index all_ctx_tiles holds the rows of this call
    const int ctx_tiles = max(0, min(tb, all_ctx_tiles) - ta);
    const int ntiles = tb - ta;
    const int k_begin = ta * TK;
    const int k_end = min(ctx, (ta + ctx_tiles) * TK);
    const int split = ta;                                            // (first block of the pair appends the new rows)

    const uint32_t sQ = smem_u32(smem);
    const uint32_t sKV = sQ + 16 * ROWB;
    const int* table = a.block_table + (size_t)b * a.max_pages;

    if (producer) {
        // ---- producer warp: keep the ring full with the tiles [ta, tb) of this pair ----
        // the math warps use the staging memory as scratch when they merge at the end of a pair: wait until the previous pair is done
        if (pairs_done > 0 && !sm100::mbar_wait(rbar(2 * ATT_STAGES), (pairs_done - 1) & 1u)) { if (lane == 0) atomicExch(a.status, 2); return; }
        pairs_done++;
        for (int t = 0; t < ntiles; t++, ring_n++) {
            const int stage = ring_n % ATT_STAGES;
            if (ring_n >= ATT_STAGES && !sm100::mbar_wait(rbar(ATT_STAGES + stage), ((ring_n / ATT_STAGES) - 1) & 1u)) { if (lane == 0) atomicExch(a.status, 2); return; }
            const uint32_t dK = sKV + stage * 2 * TILE_BYTES, dV = dK + TILE_BYTES;
            if (t < ctx_tiles) {
                if (lane == 0) {
                    const int key = k_begin + t * TK;
                    int page = table[key / a.page_size];
                    if (page < 0 || page >= a.n_pages) { atomicExch(a.status, 1); page = 0; }
                    const int row = key % a.page_size;
                    sm100::mbar_expect_tx(rbar(stage), 2 * TILE_BYTES);
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                                     ::"r"(dK + j * 8192), "l"(&tmK), "r"(rbar(stage)), "r"(64 * j), "r"(row), "r"(kvh), "r"(page) : "memory");
                        asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                                     ::"r"(dV + j * 8192), "l"(&tmV), "r"(rbar(stage)), "r"(64 * j), "r"(row), "r"(kvh), "r"(page) : "memory");
                    }
                }
            } else {
                // the rows of this call: copied from k_new / v_new by the 32 lanes; V rows M..15 are zeroed (key group 0 reads 16 rows)
                for (int i = lane; i < 16 * 32; i += 32) {
                    const int r = i >> 5, c = i & 31;
                    uint4 kv4 = make_uint4(0, 0, 0, 0), vv4 = make_uint4(0, 0, 0, 0);
                    if (r < M) {
                        const size_t off = (((size_t)b * M + r) * ATT_KV + kvh) * ATT_D;
                        kv4 = reinterpret_cast<const uint4*>(a.k_new + off)[c];
                        vv4 = reinterpret_cast<const uint4*>(a.v_new + off)[c];
                    }
                    *reinterpret_cast<uint4*>(smem + 16 * ROWB + stage * 2 * TILE_BYTES + swz_t(r, c)) = kv4;
                    *reinterpret_cast<uint4*>(smem + 16 * ROWB + stage * 2 * TILE_BYTES + TILE_BYTES + swz_t(r, c)) = vv4;
                }
                sm100::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) sm100::mbar_arrive(rbar(stage));
            }
        }
        continue;
    }
    // ---- append the new rows to the cache (first split only; readers take them from the inputs) ----
    if (split == 0) {
        for (int i = tid; i < M * 64; i += ATT_THREADS) {
            const int jj = i >> 6, c = i & 31, isv = (i >> 5) & 1;
            const int pos = ctx + jj;
            const int page = table[pos / a.page_size];
            if (page < 0 || page >= a.n_pages) { atomicExch(a.status, 1); continue; }
            const __nv_bfloat16* src = (isv ? a.v_new : a.k_new) + (((size_t)b * M + jj) * ATT_KV + kvh) * ATT_D;
            __nv_bfloat16* dst = (isv ? a.v_pages : a.k_pages) + (((size_t)page * ATT_KV + kvh) * a.page_size + pos % a.page_size) * ATT_D;
            reinterpret_cast<uint4*>(dst)[c] = reinterpret_cast<const uint4*>(src)[c];
        }
    }

    // ---- Q rows: row r = j*4 + hq  <->  q[(b*M + j), kvh*4 + hq, :]; rows >= 4M are zero ----
    for (int i = tid; i < 16 * 32; i += ATT_THREADS) {
        const int r = i >> 5, c = i & 31, j = r >> 2, hq = r & 3;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (j < M) v = reinterpret_cast<const uint4*>(a.q + (((size_t)b * M + j) * ATT_H + kvh * ATT_GQA + hq) * ATT_D)[c];
        *reinterpret_cast<uint4*>(smem + swz(r, c)) = v;
    }

    // element offset of every key row of a tile (or -1 = zero fill), looked up once per tile by threads 0..63
    long long* row_off = reinterpret_cast<long long*>(smem + 16 * ROWB + ATT_STAGES * 2 * TILE_BYTES);
    auto plan_tile = [&](int t, int stage) {
        if (tid < TK) {
            long long off = -1;
            if (t < ctx_tiles) {
                const int key = k_begin + t * TK + tid;
                if (key < k_end) {
                    int page = table[key / a.page_size];
                    // a corrupt table entry is reported and page 0 is read in its place (in bounds; that sequence's output is undefined)
                    if (page < 0 || page >= a.n_pages) { atomicExch(a.status, 1); page = 0; }
                    off = (((long long)page * ATT_KV + kvh) * a.page_size + key % a.page_size) * ATT_D;
                }
            } else if (tid < M) {
                off = -2 - ((((long long)b * M + tid) * ATT_KV + kvh) * ATT_D);          // new rows live in k_new / v_new
            }
            row_off[stage * TK + tid] = off;
        }
    };
    auto load_tile = [&](int stage) {
        const int c = tid & 31;
        // rows warp, warp + 8, ...: r & 7 is the same for all of them, so the swizzled chunk offset is a per-thread constant
        const uint32_t dK = sKV + stage * 2 * TILE_BYTES + swz(tid >> 5, c), dV = dK + TILE_BYTES;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int r = (tid >> 5) + 8 * i;
            const long long off = row_off[stage * TK + r];
            const __nv_bfloat16 *srcK = a.k_pages, *srcV = a.v_pages;
            int bytes = 0;
            if (off >= 0) { srcK = a.k_pages + off; srcV = a.v_pages + off; bytes = 16; }
            else if (off <= -2) { srcK = a.k_new + (-2 - off); srcV = a.v_new + (-2 - off); bytes = 16; }
            cp_async16(dK + i * 8 * ROWB, reinterpret_cast<const uint4*>(srcK) + (bytes ? c : 0), bytes);
            cp_async16(dV + i * 8 * ROWB, reinterpret_cast<const uint4*>(srcV) + (bytes ? c : 0), bytes);
        }
    };

    const int kg = warp & 3, dh = warp >> 2;                 // key group (16 keys of a tile) and half of the head dim of this warp
    float o[16][4];
#pragma unroll
    for (int n = 0; n < 16; n++) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float sc = 0.0625f * 1.4426950408889634f;          // 256^-1/2 (qwen35/batch.py:176), scores kept in log2 units

    // prologue: plan the first three tiles, start the first two
    if (!TMA) {
        for (int t = 0; t < ATT_STAGES && t < ntiles; t++) plan_tile(t, t);
        __syncthreads();
        for (int t = 0; t < ATT_STAGES - 1; t++) {
            if (t < ntiles) load_tile(t);
            cp_async_commit();
        }
    } else {
        csync();                                                     // Q rows are in place
    }
    bool ring_ok = true;
    for (int t = 0; t < ntiles; t++) {
        const int stage = TMA ? (int)(ring_n % ATT_STAGES) : t % ATT_STAGES;
        if (!TMA) {
            // tile t+2 goes into the stage that tile t-1 used (all warps left it at the barrier that ended iteration t-1)
            if (t + ATT_STAGES - 1 < ntiles) load_tile((t + ATT_STAGES - 1) % ATT_STAGES);
            cp_async_commit();
            cp_async_wait<ATT_STAGES - 1>();
            __syncthreads();
        } else {
            ring_ok = ring_ok && sm100::mbar_wait(rbar(stage), (ring_n / ATT_STAGES) & 1u);
        }

        const bool new_tile = t >= ctx_tiles;
        const int key0 = new_tile ? 0 : k_begin + t * TK;               // position of the tile's first key in its own numbering
        const int limit = new_tile ? M : k_end - key0;                   // keys of the tile that exist
        if (kg * KPW < limit) {
            const uint32_t tK = sKV + stage * 2 * TILE_BYTES, tV = tK + TILE_BYTES;
            auto kvoff = [&](int r, int c) -> uint32_t { return TMA ? swz_t(r, c) : swz(r, c); };
            if (TMA && !new_tile && limit < kg * KPW + KPW) {
                // the tensor-map copy brought whole 64-key boxes: value rows past the end of the context hold whatever the page
                // holds there and must not reach the MMA (0 x NaN); both warps of the key group write the same zeros
                for (int i = lane; i < (kg * KPW + KPW - limit) * 32; i += 32)
                    *reinterpret_cast<uint4*>(smem + 16 * ROWB + stage * 2 * TILE_BYTES + TILE_BYTES + swz_t(limit + (i >> 5), i & 31)) = make_uint4(0, 0, 0, 0);
                sm100::fence_proxy_async_smem();                     // these generic writes precede the next tensor-map copy into the stage
                __syncwarp();
            }
            // scores of this warp's 8 keys (16 kg + 8 dh ..): one K fragment load covers two 16-dim steps
            float sc2[2][4];
            {
                // four independent accumulators: the sixteen 16-dim steps form four chains of four dependent MMAs instead of one of sixteen
                float acc4[4][4];
#pragma unroll
                for (int i = 0; i < 4; i++) { acc4[i][0] = acc4[i][1] = acc4[i][2] = acc4[i][3] = 0.f; }
#pragma unroll
                for (int kp = 0; kp < 8; kp++) {
                    uint32_t bfr[4], af[4];
                    ldsm_x4(tK + kvoff(kg * KPW + 8 * dh + (lane & 7), 4 * kp + (lane >> 3)), bfr);
                    ldsm_x4(sQ + swz((lane & 7) + 8 * ((lane >> 3) & 1), 4 * kp + (lane >> 4)), af);
                    mma_bf16(acc4[(2 * kp) & 3], af, bfr[0], bfr[1]);
                    ldsm_x4(sQ + swz((lane & 7) + 8 * ((lane >> 3) & 1), 4 * kp + 2 + (lane >> 4)), af);
                    mma_bf16(acc4[(2 * kp + 1) & 3], af, bfr[2], bfr[3]);
                }
                float own[4];
#pragma unroll
                for (int e = 0; e < 4; e++) own[e] = (acc4[0][e] + acc4[1][e]) + (acc4[2][e] + acc4[3][e]);
                // swap with the partner warp (same key group, other half of the dims): it holds the group's other 8 keys
                float4* xb = reinterpret_cast<float4*>(smem + 16 * ROWB + ATT_STAGES * 2 * TILE_BYTES + ATT_STAGES * TK * 8) + ((t & 1) * KGROUPS + kg) * 64;
                xb[dh * 32 + lane] = make_float4(own[0], own[1], own[2], own[3]);
                asm volatile("bar.sync %0, 64;" ::"r"(2 + kg) : "memory");
                const float4 oth = xb[(dh ^ 1) * 32 + lane];
                const float ot[4] = {oth.x, oth.y, oth.z, oth.w};
#pragma unroll
                for (int e = 0; e < 4; e++) { sc2[0][e] = dh ? ot[e] : own[e]; sc2[1][e] = dh ? own[e] : ot[e]; }
            }
            // mask + online softmax; thread holds rows g (e = 0,1) and g + 8 (e = 2,3), keys 16*kg + 8n + 2*t4 + (e & 1)
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int n = 0; n < 2; n++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int kk = kg * KPW + 8 * n + 2 * t4 + (e & 1);
                    const int row = g + 8 * (e >> 1);
                    const bool ok = new_tile ? (kk < M && kk <= (row >> 2)) : (kk < limit);
                    sc2[n][e] = ok ? sc2[n][e] * sc : -INFINITY;
                    mx[e >> 1] = fmaxf(mx[e >> 1], sc2[n][e]);
                }
            float alpha[2];
#pragma unroll
            for (int h = 0; h < 2; h++) {
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
                const float mn = fmaxf(m_run[h], mx[h]);
                alpha[h] = (mn == -INFINITY) ? 1.f : exp2f(m_run[h] - mn);
                m_run[h] = mn;
                l_run[h] *= alpha[h];
            }
            uint32_t pf[4], pl[4];
            {
                float p[2][4];
#pragma unroll
                for (int n = 0; n < 2; n++)
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const float mn = m_run[e >> 1];
                        p[n][e] = (mn == -INFINITY) ? 0.f : exp2f(sc2[n][e] - mn);
                        l_run[e >> 1] += p[n][e];
                    }
                pf[0] = pack_bf16x2(p[0][0], p[0][1]); pf[1] = pack_bf16x2(p[0][2], p[0][3]);
                pf[2] = pack_bf16x2(p[1][0], p[1][1]); pf[3] = pack_bf16x2(p[1][2], p[1][3]);
                // low parts: p - bf16(p), exact in fp32, then rounded to bf16 (16 significand bits in total)
#pragma unroll
                for (int n = 0; n < 2; n++)
#pragma unroll
                    for (int e = 0; e < 4; e++) p[n][e] -= bf(p[n][e]);
                pl[0] = pack_bf16x2(p[0][0], p[0][1]); pl[1] = pack_bf16x2(p[0][2], p[0][3]);
                pl[2] = pack_bf16x2(p[1][0], p[1][1]); pl[3] = pack_bf16x2(p[1][2], p[1][3]);
            }
            // the running maximum rarely moves after the first tiles: skip the rescale of the accumulators when no lane needs it
            if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
                for (int n = 0; n < 16; n++) { o[n][0] *= alpha[0]; o[n][1] *= alpha[0]; o[n][2] *= alpha[1]; o[n][3] *= alpha[1]; }
            }
#pragma unroll
            for (int nb = 0; nb < 8; nb++) {
                uint32_t vf[4];
                ldsm_x4_t(tV + kvoff(kg * KPW + (lane & 7) + 8 * ((lane >> 3) & 1), 2 * (8 * dh + nb) + (lane >> 4)), vf);
                mma_bf16(o[2 * nb], pf, vf[0], vf[1]);
                mma_bf16(o[2 * nb + 1], pf, vf[2], vf[3]);
                mma_bf16(o[2 * nb], pl, vf[0], vf[1]);
                mma_bf16(o[2 * nb + 1], pl, vf[2], vf[3]);
            }
        }
        if (!TMA) {
            // this tile's row offsets were consumed two iterations ago: plan tile t+3 into the same slot; the barrier below orders
            // the plan before the load at the top of iteration t+1
            if (t + ATT_STAGES < ntiles) plan_tile(t + ATT_STAGES, stage);
            __syncthreads();
        } else {
            __syncwarp();
            if (lane == 0) sm100::mbar_arrive(rbar(ATT_STAGES + stage));       // this warp has finished reading the stage
            ring_n++;
        }
    }
    if (!TMA) cp_async_wait<0>();
    if (TMA && !ring_ok && tid == 0) atomicExch(a.status, 2);
    csync();

    // ---- merge the four key groups (each saw a different quarter of every tile) through shared memory ----
    float* mO = reinterpret_cast<float*>(smem + 16 * ROWB);              // [4][16][256]
    float* mML = mO + KGROUPS * 16 * ATT_D;                              // [4][16][2]
#pragma unroll
    for (int h = 0; h < 2; h++) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
#pragma unroll
    for (int n = 0; n < 16; n++) {
        float* p0 = mO + ((kg * 16 + g) * ATT_D) + 128 * dh + 8 * n + 2 * t4;
        *reinterpret_cast<float2*>(p0) = make_float2(o[n][0], o[n][1]);
        *reinterpret_cast<float2*>(p0 + 8 * ATT_D) = make_float2(o[n][2], o[n][3]);
    }
    if (t4 == 0 && dh == 0) {
        mML[(kg * 16 + g) * 2] = m_run[0]; mML[(kg * 16 + g) * 2 + 1] = l_run[0];
        mML[(kg * 16 + g + 8) * 2] = m_run[1]; mML[(kg * 16 + g + 8) * 2 + 1] = l_run[1];
    }
    csync();
    const int* pbase = meta_base(a.meta, P);
    const int nsp = pbase[pair + 1] - pbase[pair];                   // blocks that share this pair
    float* part = a.part + (size_t)slot * PART_STRIDE;
    __nv_bfloat16* out_pair = a.out + ((size_t)b * M * ATT_H + kvh * ATT_GQA) * ATT_D;     // row r = j*4 + hq -> out[(b*M + j), kvh*4 + hq]
    for (int r = 0; r < 4 * M; r++) {
        float mw[KGROUPS], mstar = -INFINITY;
#pragma unroll
        for (int w = 0; w < KGROUPS; w++) { mw[w] = mML[(w * 16 + r) * 2]; mstar = fmaxf(mstar, mw[w]); }
        float wgt[KGROUPS], lsum = 0.f;
#pragma unroll
        for (int w = 0; w < KGROUPS; w++) { wgt[w] = (mw[w] == -INFINITY) ? 0.f : exp2f(mw[w] - mstar); lsum += wgt[w] * mML[(w * 16 + r) * 2 + 1]; }
        const int d = tid;                                               // 256 threads = 256 dims
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < KGROUPS; w++) acc += wgt[w] * mO[(w * 16 + r) * ATT_D + d];
        if (nsp == 1) {                                                  // the whole pair was this block's: no partial, no merge
            const float inv = lsum == 0.f ? 1.f : 1.f / lsum;          // sum == 0 guard as qwen35/batch.py:216
            out_pair[((size_t)(r >> 2) * ATT_H + (r & 3)) * ATT_D + d] = __float2bfloat16_rn(acc * inv);
        } else {
            part[r * ATT_D + d] = acc;
            if (tid == 0) { part[16 * ATT_D + 2 * r] = mstar; part[16 * ATT_D + 2 * r + 1] = lsum; }
        }
    }
    if (nsp > 1) {
        // the block that writes the last partial of a pair merges them (the counters were zeroed by this call's plan kernel)
        __shared__ int s_last;
        __threadfence();
        csync();
        if (tid == 0) s_last = atomicAdd(meta_count(a.meta, P) + pair, 1) == nsp - 1;
        csync();
        if (s_last) {
            __threadfence();
            const float* pb = a.part + (size_t)pbase[pair] * PART_STRIDE;
            // weights of every (row, partial) first (the staging memory is free here), then 16 independent accumulators per thread
            float* wsm = mO;                                             // [nsp][16] weights, then [16] 1 / sum
            for (int i = tid; i < nsp * 16; i += ATT_THREADS) wsm[i] = __ldcg(pb + (size_t)(i >> 4) * PART_STRIDE + 16 * ATT_D + 2 * (i & 15));
            csync();
            if (tid < 16) {
                float ms = -INFINITY, lsum = 0.f;
                for (int sp = 0; sp < nsp; sp++) ms = fmaxf(ms, wsm[sp * 16 + tid]);
                for (int sp = 0; sp < nsp; sp++) {
                    const float m = wsm[sp * 16 + tid];
                    const float w = (m == -INFINITY) ? 0.f : exp2f(m - ms);
                    lsum += w * __ldcg(pb + (size_t)sp * PART_STRIDE + 16 * ATT_D + 2 * tid + 1);
                    wsm[sp * 16 + tid] = w;
                }
                wsm[nsp * 16 + tid] = lsum == 0.f ? 1.f : 1.f / lsum;   // sum == 0 guard as qwen35/batch.py:216
            }
            csync();
            float acc[16];
#pragma unroll
            for (int r = 0; r < 16; r++) acc[r] = 0.f;
            for (int sp = 0; sp < nsp; sp++) {
                const float* pp = pb + (size_t)sp * PART_STRIDE + tid;
#pragma unroll
                for (int r = 0; r < 16; r++)
                    if (r < 4 * M) acc[r] += wsm[sp * 16 + r] * __ldcg(pp + r * ATT_D);
            }
#pragma unroll
            for (int r = 0; r < 16; r++)
                if (r < 4 * M) out_pair[((size_t)(r >> 2) * ATT_H + (r & 3)) * ATT_D + tid] = __float2bfloat16_rn(acc[r] * wsm[nsp * 16 + r]);
        }
    }
    if (TMA) sm100::fence_proxy_async_smem();                        // merge scratch was written through the generic proxy
    csync();                                                         // shared memory is reused by the block's next pair
    if (TMA) { __syncwarp(); if (lane == 0) sm100::mbar_arrive(rbar(2 * ATT_STAGES)); }       // the producer may refill the ring
  }
}

// ---- host side ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// pages [n_pages, 2, page_size, 256] bf16 as a 4-D tensor (256, page_size, 2, n_pages); box = 64 dims x 64 keys, 128-byte swizzle
static bool make_page_map(CUtensorMap* m, const void* base, int page_size, int n_pages) {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        cudaDriverEntryPointQueryResult qr;
        void* p = nullptr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) != cudaSuccess || qr != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            return false;
        }
        fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    const cuuint64_t dims[4] = {(cuuint64_t)ATT_D, (cuuint64_t)page_size, (cuuint64_t)ATT_KV, (cuuint64_t)n_pages};
    const cuuint64_t strides[3] = {(cuuint64_t)ROWB, (cuuint64_t)page_size * ROWB, (cuuint64_t)ATT_KV * page_size * ROWB};
    const cuuint32_t box[4] = {64, 64, 1, 1}, es[4] = {1, 1, 1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int sm_count() {
    static int sms[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return 148; }
    if (!sms[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) { cudaGetLastError(); n = 148; }
        sms[dev] = n;
    }
    return sms[dev];
}

// workspace = plan (ints) + one partial per (block, pair) intersection: at most blocks + pairs of them
size_t gqa_workspace_bytes(int B, int max_ctx) {
    (void)max_ctx;
    const int P = B * ATT_KV;
    return meta_ints(P) * sizeof(int) + (size_t)(sm_count() + P) * PART_STRIDE * sizeof(float);
}

static int launch_with_workspace(AttnArgs a, void* ws, size_t ws_bytes, const char* who, cudaStream_t stream) {
    a.P = a.B * ATT_KV;
    const size_t meta_b = meta_ints(a.P) * sizeof(int);
    const long long slots = ws_bytes > meta_b ? (long long)((ws_bytes - meta_b) / (PART_STRIDE * sizeof(float))) : 0;
    a.G = sm_count();
    if (slots - a.P < a.G) a.G = (int)(slots - a.P);                 // a smaller workspace is served with fewer blocks
    if (a.G < 1) {
        set_error("%s: scratch of %zu bytes cannot hold the plan and %d + 1 partials of %zu bytes", who, ws_bytes, a.P,
                  (size_t)PART_STRIDE * sizeof(float));
        return GDN_E_SHAPE;
    }
    a.meta = static_cast<int*>(ws);
    a.part = reinterpret_cast<float*>(static_cast<char*>(ws) + meta_b);
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        if (cudaFuncSetAttribute(gqa_decode_split_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM) != cudaSuccess ||
            cudaFuncSetAttribute(gqa_decode_split_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM) != cudaSuccess)
            return check_launch("gqa_decode smem attribute");
        attr_set[dev] = true;
    }
    // pages that hold a multiple of 64 keys: every 64-key tile lies inside one page and can be fetched by tensor-map copies
    CUtensorMap tk, tv;
    memset(&tk, 0, sizeof(tk));
    memset(&tv, 0, sizeof(tv));
    bool tma = a.page_size % TK == 0 && make_page_map(&tk, a.k_pages, a.page_size, a.n_pages) && make_page_map(&tv, a.v_pages, a.page_size, a.n_pages);
    if (tma && a.P <= TC_MAX_PAIRS) {                                // tcgen05 path: plans for itself
        a.tail_tiles = 2;
        return launch_gqa_decode_tc(a, tk, tv, stream);
    }
    a.tail_tiles = 0;
    gqa_decode_plan_kernel<<<1, 256, 0, stream>>>(a);
    int rc = check_launch("gqa_decode_plan");
    if (rc) return rc;
    if (tma) gqa_decode_split_kernel<true><<<a.G, ATT_THREADS + 32, ATT_SMEM, stream>>>(a, tk, tv);
    else gqa_decode_split_kernel<false><<<a.G, ATT_THREADS, ATT_SMEM, stream>>>(a, tk, tv);
    return check_launch("gqa_decode_split");
}

int launch_gqa_decode(AttnArgs a, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    if (a.B <= 0) return GDN_OK;
    return launch_with_workspace(a, workspace, workspace_bytes, "gqa_decode_paged", stream);
}

// ----------------------------------------------------------------------------------------------------------------------
// Variant for callers that cannot allocate device memory: the plan and the partials go to a fixed array that lives in the
// library image instead of a caller-provided workspace.  Every GPU that loads the library holds these 12 MiB until the process
// exits.  The array is shared by all calls on a device and keeps whatever the last call left in it; nothing in it has to start
// at zero (the plan kernel of a call rewrites the plan, and every partial that a merging block reads was written by the split
// kernel of the same call), but two calls that overlap on the GPU (different streams) would overwrite each other's data.
// ----------------------------------------------------------------------------------------------------------------------
constexpr int STATIC_PARTIALS = 762;                                   // partial slots that fit next to the plan
constexpr int STATIC_MAX_B = 256;                                      // sequences per call: 2 * 256 pairs + one block per SM <= 762
constexpr size_t STATIC_SCRATCH_FLOATS = (size_t)STATIC_PARTIALS * PART_STRIDE + meta_ints(2 * STATIC_MAX_B);      // partials + the plan of 512 pairs
static __device__ __align__(256) float g_static_scratch[STATIC_SCRATCH_FLOATS];                                    // 12 MiB

int launch_gqa_decode_static(AttnArgs a, cudaStream_t stream) {
    if (a.B <= 0) return GDN_OK;
    if (a.B > STATIC_MAX_B) {
        set_error("gqa_decode_paged_static: B=%d sequences exceed the %d the built-in scratch is sized for (%d partial slots; "
                  "use gqa_decode_paged with a workspace of gqa_decode_workspace_bytes() instead)", a.B, STATIC_MAX_B, STATIC_PARTIALS);
        return GDN_E_SHAPE;
    }
    // In host code the array's name is only a handle: the device address has to be asked for, once per device, with that device
    // current.  The first call on a device does it (and should therefore come before any stream capture).
    static float* addr[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return check_launch("gqa_decode_paged_static: device");
    if (!addr[dev]) {
        float* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_scratch);
        if (e != cudaSuccess || !p) {
            cudaGetLastError();
            set_error("gqa_decode_paged_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return GDN_E_LAUNCH;
        }
        addr[dev] = p;
    }
    return launch_with_workspace(a, addr[dev], sizeof(float) * STATIC_SCRATCH_FLOATS, "gqa_decode_paged_static", stream);
}

}  // namespace gdn
