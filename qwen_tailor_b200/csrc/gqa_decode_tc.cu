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
// Roles (128 threads, one persistent block per SM): warp 0 softmax / epilogue (lanes r and r + 16 share query row r), warp 1 lane 0
// issues the MMAs, warp 2 is the TMA producer (three-stage ring of K + V tiles; it runs ahead on its own through all the pairs of
// the block's range, and marks the cache lines evict-first so that the stream does not flush everything else out of L2), warp 3
// stages Q and appends the new rows -- for the block's next pair while the current one streams, because a plain load issued
// while the copies saturate the memory system takes microseconds.
//
// There is no plan kernel in front of this one: every block derives the balanced split from the context lengths itself.  The
// blocks of a pair meet at an arrival counter in the workspace; the one that arrives last merges the pair's partials, which it
// fetches with bulk copies into the (then idle) ring when the pair is the block's last.  The counters carry an epoch tag and need
// no zeroing, see `touch` / `arrive` below.
// Every wait is bounded; a wait that gives up sets the device status word and the block runs out its loops without touching
// the tensor cores again.
#include <cstring>
#include "gqa_common.cuh"
#include "sm100_prims.cuh"

namespace gdn {

using namespace sm100;

constexpr uint32_t TCM_O = 0, TCM_S0 = 256, TCM_P0 = 384;            // O [256], S buffers [64] x 2, P buffers [hi 32 | lo 32] x 2
enum { TB_FULL0 = 0, TB_EMPTY0 = 3, TB_SDONE0 = 6, TB_SFREE0 = 8, TB_PREADY0 = 10, TB_PFREE0 = 12, TB_ODONE = 14, TB_MERGE = 15, TB_COUNT = 16 };
constexpr int TC_RING_PARTIALS = ATT_STAGES * 2 * TILE_BYTES / (PART_STRIDE * 4);      // partial images the idle ring can hold (11)
constexpr float TC_RESCALE_STEP = 8.f;                               // log2 units

// Weighted sum of the partials of a pair (the standard split-softmax merge): nsp images of PART_STRIDE floats at pb, in global
// memory (read through L2) or, SM = true, already copied into shared memory.  Run by the 96 consumer threads.
template <bool SM>
__device__ __forceinline__ void tc_merge_pair(const float* pb, int nsp, float* s_w, float* s_l, __nv_bfloat16* out_pair, int M, int ctid) {
    auto csync = [&]() { asm volatile("bar.sync 1, 96;" ::: "memory"); };
    for (int i = ctid; i < nsp * 16; i += 96) {
        const float2* src = reinterpret_cast<const float2*>(pb + (size_t)(i >> 4) * PART_STRIDE + 16 * ATT_D + 2 * (i & 15));
        const float2 ml = SM ? *src : __ldcg(src);
        s_w[i] = ml.x;
        s_l[i] = ml.y;
    }
    csync();
    {
        // weights: thread (row, group of partials) -- six threads share a row's partials, the row's maximum and sum go through s_red
        const int r = ctid & 15, g = ctid >> 4;
        float* s_red = s_l + nsp * 16;                               // [6][16] maxima, then [6][16] sums
        float mx = -INFINITY;
        for (int sp = g; sp < nsp; sp += 6) mx = fmaxf(mx, s_w[sp * 16 + r]);
        s_red[g * 16 + r] = mx;
        csync();
        float ms = s_red[r];
#pragma unroll
        for (int k = 1; k < 6; k++) ms = fmaxf(ms, s_red[k * 16 + r]);
        float lsum = 0.f;
        for (int sp = g; sp < nsp; sp += 6) {
            const float m = s_w[sp * 16 + r];
            const float w = (m == -INFINITY) ? 0.f : exp2f(m - ms);
            lsum += w * s_l[sp * 16 + r];
            s_w[sp * 16 + r] = w;
        }
        s_red[96 + g * 16 + r] = lsum;
        csync();
        if (g == 0) {
            float t = 0.f;
#pragma unroll
            for (int k = 0; k < 6; k++) t += s_red[96 + k * 16 + r];
            s_w[nsp * 16 + r] = t == 0.f ? 1.f : 1.f / t;            // sum == 0 guard as qwen35/batch.py:216
        }
    }
    csync();
    GDN_BSTAMP(15);
    // thread = (row, four dims), four of them at a time (independent loads and sums): neighbouring threads read neighbouring
    // 16-byte words, every partial is an independent load
    const int n_out = 4 * M * 64;
    for (int k0 = 0; k0 * 96 < n_out; k0 += 4) {
        float4 acc[4];
        int r[4];
        const float* col[4];
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const int idx = min(ctid + 96 * (k0 + q), n_out - 1);
            r[q] = idx >> 6;
            col[q] = pb + r[q] * ATT_D + (idx & 63) * 4;
            acc[q] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll 2
        for (int sp = 0; sp < nsp; sp++) {
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float4* src = reinterpret_cast<const float4*>(col[q] + (size_t)sp * PART_STRIDE);
                const float4 x = SM ? *src : __ldcg(src);
                const float w = s_w[sp * 16 + r[q]];
                acc[q].x += w * x.x; acc[q].y += w * x.y; acc[q].z += w * x.z; acc[q].w += w * x.w;
            }
        }
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const int idx = ctid + 96 * (k0 + q);
            if (idx < n_out) {
                const float inv = s_w[nsp * 16 + r[q]];
                uint2 v;
                v.x = pack_bf16x2(acc[q].x * inv, acc[q].y * inv);
                v.y = pack_bf16x2(acc[q].z * inv, acc[q].w * inv);
                *reinterpret_cast<uint2*>(out_pair + ((size_t)(r[q] >> 2) * ATT_H + (r[q] & 3)) * ATT_D + (idx & 63) * 4) = v;
            }
        }
    }
}

__global__ void __launch_bounds__(TC_THREADS, 1)
gqa_decode_tc_kernel(const AttnArgs a, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV) {
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ uint64_t bars[TB_COUNT];
    __shared__ uint32_t tmem_slot;
    __shared__ int s_abort, s_last;
    __shared__ float s_w[(148 + 2) * 16];                            // merge weights: [partials of a pair][16 rows], then 1 / sum
    __shared__ int s_cum[TC_MAX_PAIRS + 1];                   // the plan: tile prefix sums of the pairs,
    __shared__ int s_base[TC_MAX_PAIRS + 1];                  //   first partial slot of every pair,
    __shared__ int s_ctx[TC_MAX_PAIRS / ATT_KV];              //   context lengths
    __shared__ int s_scan[TC_THREADS / 32];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int M = a.M, P = a.P;
    const uint32_t sbase = smem_addr(smem);
    if (sbase & 1023u) { if (tid == 0) atomicExch(a.status, 4); return; }
    // Programmatic dependent launch: the next kernel of the stream may be scheduled onto SMs as this one leaves them, and this one
    // waits here -- before it reads anything an earlier kernel may have written -- until its predecessors have completed.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- the plan, computed by every block for itself (a few hundred integer operations; a kernel of its own in front of this one
    //      costs a launch and a dependent start per layer).  Same plan as gqa_decode_plan_kernel: the tiles of all pairs laid end to
    //      end, every pair followed by `tail_tiles` tiles of weight without work, cut into G equal ranges. ----
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(a.meta + 2);
    for (int i = tid; i < a.B; i += TC_THREADS) s_ctx[i] = a.ctx_len[i];
    __syncthreads();
    const int* cum = s_cum;
    const int* ctxv = s_ctx;
    auto block_scan = [&](int local) -> int {                        // exclusive prefix of `local` over the block
        int x = local;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const int y = __shfl_up_sync(0xffffffffu, x, o); if (lane >= o) x += y; }
        __syncthreads();
        if (lane == 31) s_scan[warp] = x;
        __syncthreads();
        int before = 0;
        for (int w = 0; w < warp; w++) before += s_scan[w];
        return before + x - local;
    };
    const int chunk = (P + TC_THREADS - 1) / TC_THREADS, p0 = min(P, tid * chunk), p1 = min(P, p0 + chunk);
    auto tiles_of = [&](int p) -> int {
        const int ctx = s_ctx[p / ATT_KV];
        if (ctx < 0 || (long long)ctx + M > (long long)a.max_pages * a.page_size) { atomicExch(a.status, 1); return 0; }
        return (ctx + TK - 1) / TK + 1 + a.tail_tiles;
    };
    {
        int local = 0;
        for (int p = p0; p < p1; p++) local += tiles_of(p);
        int run = block_scan(local);
        for (int p = p0; p < p1; p++) { s_cum[p] = run; run += tiles_of(p); }
        if (tid == TC_THREADS - 1) s_cum[P] = run;                   // (the last thread's chunk ends the range, or is empty: run = total)
    }
    __syncthreads();
    const long long N = s_cum[P];
    // with fewer tiles than blocks only the first N blocks work (one tile each): every working block then has a non-empty range
    const int G = (int)min((long long)gridDim.x, max(N, 1ll));
    auto first_block = [&](int p) -> int { return block_of_tile(s_cum[p], G, N); };
    auto partials_of = [&](int p) -> int {                           // blocks that hold tiles with work of pair p (consecutive)
        return s_cum[p + 1] > s_cum[p] ? block_of_tile(s_cum[p + 1] - 1 - a.tail_tiles, G, N) - first_block(p) + 1 : 0;
    };
    {
        int local = 0;
        for (int p = p0; p < p1; p++) local += partials_of(p);
        int run = block_scan(local);
        for (int p = p0; p < p1; p++) { s_base[p] = run; run += partials_of(p); }
        if (tid == TC_THREADS - 1) s_base[P] = run;
    }
    __syncthreads();
    if ((int)blockIdx.x >= G || N == 0) return;
    long long lo = (long long)blockIdx.x * N / G;
    const long long hi = (long long)(blockIdx.x + 1) * N / G;
    // Arrival counters in the workspace: 64-bit words {tag, count}, valid only while the tag is the one of this call's epoch; the
    // block that arrives last at the end of the kernel advances the epoch word, which invalidates every counter at once.  Nothing
    // has to be zeroed between calls, and whatever an allocator left in the workspace reads as "no arrivals yet".  A block first
    // `touch`es a counter it will arrive at (long before it does: if the word is stale, one compare-and-swap -- whoever wins --
    // makes it {tag, 0}); the arrival itself is then a plain atomic add.
    unsigned long long* counters = reinterpret_cast<unsigned long long*>(a.meta + 4);      // [0] blocks done, [1 + p] partials of pair p
    auto tag_of = [&](int idx) -> uint32_t { return epoch * 0x9E3779B1u + (uint32_t)idx + 1u; };
    auto touch = [&](int idx) {
        const unsigned long long v = *reinterpret_cast<volatile unsigned long long*>(counters + idx);
        if ((uint32_t)(v >> 32) != tag_of(idx)) atomicCAS(counters + idx, v, (unsigned long long)tag_of(idx) << 32);
    };
    auto arrive = [&](int idx) -> uint32_t { return (uint32_t)atomicAdd(counters + idx, 1ull); };      // how many arrived before
    if (tid == 0) touch(0);
    auto bar = [&](int i) -> uint32_t { return smem_addr(&bars[i]); };
    if (tid == 0) {
        for (int i = 0; i < 3; i++) { mbar_init(bar(TB_FULL0 + i), 1); mbar_init(bar(TB_EMPTY0 + i), 1); }
        for (int i = 0; i < 2; i++) { mbar_init(bar(TB_SDONE0 + i), 1); mbar_init(bar(TB_SFREE0 + i), 1); mbar_init(bar(TB_PREADY0 + i), 1); mbar_init(bar(TB_PFREE0 + i), 1); }
        mbar_init(bar(TB_ODONE), 1);
        mbar_init(bar(TB_MERGE), 1);
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
    int pair;                                                        // pair that owns tile lo: cum[pair] <= lo < cum[pair + 1]
    {
        int l = 0, r = P - 1;
        while (l < r) { const int m = (l + r + 1) >> 1; if (cum[m] <= lo) l = m; else r = m - 1; }
        pair = l;
    }
    // work of this block in pair pr, from tile l on: the tiles past the pair's last real one are the plan's weight of its epilogue
    auto seg_tiles = [&](int pr, long long l) -> int {
        const int ta = (int)(l - cum[pr]), tbk = (int)(min(hi, (long long)cum[pr + 1]) - cum[pr]);
        return max(0, min(tbk, (ctxv[pr / ATT_KV] + TK - 1) / TK + 1) - ta);
    };
    auto next_seg = [&](int pr, long long l, int& npair, int& nta) -> bool {      // first segment with work after (pr, l); l = its start
        for (pr++; l < hi; pr++) {
            if (cum[pr + 1] <= l) continue;
            if (seg_tiles(pr, l) > 0) { npair = pr; nta = (int)(l - cum[pr]); return true; }
            l = min(hi, (long long)cum[pr + 1]);
        }
        return false;
    };
    // the three consumer warps synchronise among themselves; the producer runs ahead on its own, across pair boundaries
    auto csync = [&]() { asm volatile("bar.sync 1, 96;" ::: "memory"); };
    const int ctid = warp < 2 ? tid : tid - 32;                      // 0..95 over warps 0, 1, 3

    if (warp == 2) {
        // ================= producer: keep the ring full with every tile of this block's range, pair after pair =================
        uint32_t n = 0;
        long long plo = lo;
        int ahead_page = 0;                                          // this lane's page number for the next segment's first 32 tiles
        bool have_pages = false;
        // the cache is read once per call: its lines are the first to leave L2, so that the plan, the page table, the partials and
        // the code stay there while hundreds of megabytes stream through
        uint64_t stream_policy;
        asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(stream_policy));
        for (int pp = pair; plo < hi && !aborted(); pp++) {
            if (cum[pp + 1] <= plo) continue;
            const long long seg_end = min(hi, (long long)cum[pp + 1]);
            const int ta = (int)(plo - cum[pp]), tbk = (int)(seg_end - cum[pp]);
            plo = seg_end;
            const int b = pp / ATT_KV, kvh = pp % ATT_KV;
            const int ctx = ctxv[b];
            const int all_ctx = (ctx + TK - 1) / TK;
            const int ctx_tiles = max(0, min(tbk, all_ctx) - ta);
            const int ntiles = max(0, min(tbk, all_ctx + 1) - ta);         // tiles past all_ctx are the plan's weight of the epilogue: no work
            bool okp = true;
            int my_page = 0;
            // page numbers, one lane per tile, 32 tiles at a time.  Those of a segment's first 32 tiles were requested while the
            // previous segment streamed (a load issued under the copies takes microseconds, and the ring only holds three tiles).
            auto pages_of = [&](int pr, int first_tile) -> int {         // this lane's page of tile first_tile + lane of pair pr
                const int pctx = ctxv[pr / ATT_KV];
                const int e = (int)(((long long)(first_tile + lane) * TK) / a.page_size);
                return (first_tile + lane < (pctx + TK - 1) / TK && e < a.max_pages) ? a.block_table[(size_t)(pr / ATT_KV) * a.max_pages + e] : 0;
            };
            int npair = 0, nta = 0;
            const bool has_next = next_seg(pp, seg_end, npair, nta);
            for (int t = 0; t < ntiles && okp; t++, n++) {
                if ((t & 31) == 0) {
                    my_page = (t == 0 && have_pages) ? ahead_page : pages_of(pp, ta + t);
                    if (t == 0) { have_pages = has_next; if (has_next) ahead_page = pages_of(npair, nta); }
                }
                int page = __shfl_sync(0xffffffffu, my_page, t & 31);
                const int stage = n % ATT_STAGES;
                if (n >= (uint32_t)ATT_STAGES && !wait(TB_EMPTY0 + stage, (n / ATT_STAGES) - 1)) { okp = false; break; }
                const uint32_t dK = sKV + stage * 2 * TILE_BYTES, dV = dK + TILE_BYTES;
                if (t < ctx_tiles) {
                    if (lane == 0) {
                        const int key = (ta + t) * TK;
                        if (page < 0 || page >= a.n_pages) { atomicExch(a.status, 1); page = 0; }      // reported; page 0 is read in its place
                        const int row = key % a.page_size;
                        mbar_expect_tx(bar(TB_FULL0 + stage), 2 * TILE_BYTES);
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5, %6}], [%2], %7;"
                                         ::"r"(dK + j * 8192), "l"(&tmK), "r"(bar(TB_FULL0 + stage)), "r"(64 * j), "r"(row), "r"(kvh), "r"(page), "l"(stream_policy) : "memory");
                            asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5, %6}], [%2], %7;"
                                         ::"r"(dV + j * 8192), "l"(&tmV), "r"(bar(TB_FULL0 + stage)), "r"(64 * j), "r"(row), "r"(kvh), "r"(page), "l"(stream_policy) : "memory");
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
            if (!okp) break;
        }
    } else {
    uint32_t n0 = 0;                                                 // tiles this block has put through the ring before the current pair
    uint32_t pairs_done = 0, merges_done = 0;                       // pairs seen; merges that went through the ring
    // warp 3 keeps the Q rows of the next pair in registers: fetched while the current pair streams (a load issued then takes
    // microseconds, the memory system being saturated by the copies), written to the operand slabs when the tensor pipe is done
    uint4 qreg[16];
    bool q_have = false;
    auto q_fetch = [&](int pr) {
        const int b = pr / ATT_KV, kvh = pr % ATT_KV;
#pragma unroll
        for (int r = 0; r < 16; r++) {
            const int j = r >> 2, hq = r & 3;
            qreg[r] = make_uint4(0, 0, 0, 0);
            if (j < M) qreg[r] = reinterpret_cast<const uint4*>(a.q + (((size_t)b * M + j) * ATT_H + kvh * ATT_GQA + hq) * ATT_D)[lane];
        }
    };
    auto q_put = [&]() {                                             // row r = j*4 + hq; rows 16..31 repeat rows 0..15; rows >= 4M zero
#pragma unroll
        for (int r = 0; r < 16; r++) {
            unsigned char* dst = smem + (lane >> 3) * 4096 + r * 128 + (((lane & 7) ^ (r & 7)) << 4);
            *reinterpret_cast<uint4*>(dst) = qreg[r];
            *reinterpret_cast<uint4*>(dst + 2048) = qreg[r];         // (r + 16 has the same r & 7)
        }
        fence_proxy_async_smem();
    };
    auto append = [&](int pr) {                                      // the rows of this call into the cache (readers take them from the inputs)
        const int b = pr / ATT_KV, kvh = pr % ATT_KV;
        const int ctx = ctxv[b];
        const int* table = a.block_table + (size_t)b * a.max_pages;
        for (int i = lane; i < M * 64; i += 32) {
            const int jj = i >> 6, c = i & 31, isv = (i >> 5) & 1;
            const int pos = ctx + jj;
            const int page = table[pos / a.page_size];
            if (page < 0 || page >= a.n_pages) { atomicExch(a.status, 1); continue; }
            const __nv_bfloat16* src = (isv ? a.v_new : a.k_new) + (((size_t)b * M + jj) * ATT_KV + kvh) * ATT_D;
            __nv_bfloat16* dst = (isv ? a.v_pages : a.k_pages) + (((size_t)page * ATT_KV + kvh) * a.page_size + pos % a.page_size) * ATT_D;
            reinterpret_cast<uint4*>(dst)[c] = reinterpret_cast<const uint4*>(src)[c];
        }
    };
    for (; lo < hi; pair++) {
        if (cum[pair + 1] <= lo) continue;                           // pairs without tiles (rejected sequences)
        if (seg_tiles(pair, lo) == 0) { lo = min(hi, (long long)cum[pair + 1]); continue; }      // only weight tiles of this pair: no partial either
        const long long seg_end = min(hi, (long long)cum[pair + 1]);
        const int ta = (int)(lo - cum[pair]), tbk = (int)(seg_end - cum[pair]);      // this block's tiles of the pair: [ta, tbk)
        const int slot = s_base[pair] + ((int)blockIdx.x - first_block(pair));
        int npair = 0, nta = 0;
        const bool has_next = next_seg(pair, seg_end, npair, nta);  // (the same answer in every thread)
        lo = seg_end;
        const int b = pair / ATT_KV, kvh = pair % ATT_KV;
        const int ctx = ctxv[b];
        const int all_ctx_tiles = (ctx + TK - 1) / TK;               // tile index all_ctx_tiles holds the rows of this call
        const int ctx_tiles = max(0, min(tbk, all_ctx_tiles) - ta);
        const int ntiles = max(0, min(tbk, all_ctx_tiles + 1) - ta);   // tiles past all_ctx_tiles are the plan's weight of the epilogue: no work
        const int k_begin = ta * TK;
        const int k_end = min(ctx, (ta + ctx_tiles) * TK);

        // ---- prologue: Q rows into the operand slabs and, in the block that owns the pair's first tile, the new rows into the cache ----
        if (warp == 3) {
            if (!q_have) { q_fetch(pair); if (ta == 0) append(pair); }
            q_put();
        }
        csync();
        if (pairs_done == 0) GDN_BSTAMP(6);

        if (warp == 1) {
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
                    if (n == 0) GDN_BSTAMP_ANY(10);
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
            if (pairs_done == 0 && lane == 0) GDN_BSTAMP_ANY(7);
            if (ok) ok = wait(TB_ODONE, pairs_done);
            tc_fence_after_sync();
            if (pairs_done == 0 && lane == 0) GDN_BSTAMP_ANY(8);
            const int nsp = s_base[pair + 1] - s_base[pair];
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
            if (pairs_done == 0 && lane == 0) GDN_BSTAMP_ANY(9);
            tc_fence_before_sync();
        } else if (warp == 3) {
            // ================= look-ahead: the next pair's Q rows (and its append) while this one streams =================
            if (lane == 0) { touch(1 + pair); __threadfence(); }     // (not on the softmax warp: under the copies this takes microseconds)
            q_have = has_next;
            if (has_next) { q_fetch(npair); if (nta == 0) append(npair); }
        }
        n0 += ntiles;
        pairs_done++;
        GDN_BSTAMP(1 + 2 * (pairs_done > 1));

        // ---- merge: the block that writes the last partial of a pair combines them (the counters were zeroed by this call's plan kernel) ----
        const int* pbase = s_base;
        const int nsp = pbase[pair + 1] - pbase[pair];
        __threadfence();
        csync();
        if (nsp > 1) {
            if (ctid == 0) s_last = (!aborted() && arrive(1 + pair) == (uint32_t)(nsp - 1)) ? 1 : 0;
            csync();
            GDN_BSTAMP(13);
            if (s_last && nsp <= 148) {
                __threadfence();
                const float* pb = a.part + (size_t)pbase[pair] * PART_STRIDE;
                float* s_l = reinterpret_cast<float*>(smem);         // the partials' sums: the Q operand is idle between pairs
                __nv_bfloat16* out_pair = a.out + ((size_t)b * M * ATT_H + kvh * ATT_GQA) * ATT_D;
                if (!has_next && nsp <= TC_RING_PARTIALS) {
                    // the block's last pair: the ring is idle, so the partials come in as bulk copies, all in flight at once (read
                    // through registers they cost several dependent round trips to L2)
                    unsigned char* ring = smem + TC_Q_BYTES;
                    if (ctid == 0) {
                        asm volatile("fence.proxy.async;" ::: "memory");
                        mbar_expect_tx(bar(TB_MERGE), (uint32_t)nsp * PART_STRIDE * 4);
                        for (int sp = 0; sp < nsp; sp++)
                            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                         ::"r"(smem_addr(ring + (size_t)sp * PART_STRIDE * 4)), "l"(pb + (size_t)sp * PART_STRIDE), "r"(PART_STRIDE * 4), "r"(bar(TB_MERGE)) : "memory");
                    }
                    const bool got = wait(TB_MERGE, merges_done);
                    GDN_BSTAMP(14);
                    if (got) tc_merge_pair<true>(reinterpret_cast<const float*>(ring), nsp, s_w, s_l, out_pair, M, ctid);
                    else { csync(); csync(); csync(); csync(); }     // (keeps the barrier count of the merge)
                    merges_done++;
                } else {
                    tc_merge_pair<false>(pb, nsp, s_w, s_l, out_pair, M, ctid);
                }
            }
            csync();                                         // s_w and s_last are reused by the block's next pair
        }
        GDN_BSTAMP(2 + 2 * (pairs_done > 1));
    }
    GDN_BVAL(11, n0); GDN_BVAL(12, pairs_done);
    }   // consumer warps
    tc_fence_before_sync();
    __syncthreads();
    GDN_BSTAMP(5);
    if (warp == 1) tmem_dealloc(tb, 512);
    // the last block to get here -- blocks that gave up on a wait come here too -- starts the next call's epoch
    if (tid == 0) {
        __threadfence();
        if (arrive(0) == (uint32_t)(G - 1)) { *reinterpret_cast<volatile uint32_t*>(a.meta + 2) = epoch + 1u; __threadfence(); }
    }
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
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)a.G); cfg.blockDim = dim3(TC_THREADS); cfg.dynamicSmemBytes = TC_SMEM; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, gqa_decode_tc_kernel, a, tk, tv);
    return check_launch("gqa_decode_tc");
}

}  // namespace gdn

#ifdef GDN_TIMING
extern "C" __attribute__((visibility("default"))) int gdn_timing_log_c(long long* out_host, int n) {
    return cudaMemcpyFromSymbol(out_host, gdn::g_tlog, sizeof(long long) * n) == cudaSuccess ? 0 : -5;
}
#endif
