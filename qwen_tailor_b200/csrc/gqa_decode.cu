// GQA decode attention, head_dim 256, 8 query heads / 2 KV heads, over a paged bf16 KV cache.
//
// Replaces the reference's `attn_b` Metal kernel (qwen35/batch.py:141-237): for row r = b*M + j, softmax(q K^T / 16) V over
// the keys [0, ctx_len[b] + j]; the keys/values of the M rows of this call are taken from the call's inputs (never from the
// cache, so the in-place append needs no ordering against readers, batch.py:143-148,182) and are appended to the cache at
// positions ctx_len[b] + j.  The reference's contiguous slot pool [S+1, 2, Lmax, 256] is the special case
// page_size = Lmax, block_table[b] = {slot}.
//
// The kernel is bound by streaming K and V once (2 KiB per cached token and layer).  Design:
//   * split-KV: grid (split, kv_head, sequence); every block streams `split_keys` keys of one (sequence, kv head) so that a
//     ragged batch still fills 148 SMs; partial (max, sum, O) go to a caller-provided fp32 workspace and a second kernel
//     merges them.
//   * GQA packing: the 4 query heads of a KV head times the M <= 4 chained rows form the 16 rows of a warp-level
//     m16n8k16 bf16 MMA, so each K/V byte is read once for up to 16 query rows (at M = 4 plain FMAs could not keep up with
//     HBM).  Each of the 8 warps owns 8 of the 64 keys of a tile (scores by m16n8k16, P.V by m16n8k8) and keeps its own
//     online-softmax state; eight warps rather than four because the per-tile dependency chains (16 chained score MMAs,
//     the softmax shuffles) are latency-bound and need other warps to hide behind.
//   * K/V tiles (64 keys x 512 B) are gathered page by page with 16-byte cp.async into XOR-swizzled shared memory, three
//     stages (192 KiB per SM, two tiles in flight while one is consumed).  The page lookup of a tile's 64 keys is done once
//     (one thread per key) and shared through shared memory.
//   * the probabilities are fed to the P.V MMA as a bf16 hi + lo pair, so the result carries fp32-level accuracy like the
//     reference's fp32 accumulation of exp_score * v.
#include "gdn_common.cuh"
#include "launchers.cuh"

namespace gdn {

constexpr int ATT_H = 8, ATT_KV = 2, ATT_D = 256, ATT_GQA = 4;
constexpr int TK = 64;                          // keys per tile
constexpr int ATT_WARPS = 8, ATT_THREADS = 256, KPW = TK / ATT_WARPS;      // 8 keys per warp
constexpr int ROWB = ATT_D * 2;                 // bytes per key row (512)
constexpr int TILE_BYTES = TK * ROWB;           // 32 KiB
constexpr int ATT_STAGES = 3;
constexpr int ATT_SMEM = 16 * ROWB + ATT_STAGES * 2 * TILE_BYTES + ATT_STAGES * TK * 8;     // Q (8 KiB) + stages x (K + V) + row offsets
constexpr int PART_STRIDE = 16 * ATT_D + 32;    // floats per (sequence, kv head, split): O[16][256] + (m, l)[16]


__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_k8(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(b0));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// byte offset of 16-byte chunk `c` of row `r` in a swizzled [rows][512 B] tile
__device__ __forceinline__ uint32_t swz(int r, int c) { return (uint32_t)(r * ROWB + ((c ^ (r & 7)) << 4)); }

__device__ __forceinline__ int n_splits_of(int ctx, int split_keys) { int n = (ctx + split_keys - 1) / split_keys; return n < 1 ? 1 : n; }

__global__ void __launch_bounds__(ATT_THREADS, 1) gqa_decode_split_kernel(const AttnArgs a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int M = a.M;
    const int ctx = a.ctx_len[b];
    if (ctx < 0 || (long long)ctx + M > (long long)a.max_pages * a.page_size) { if (tid == 0) atomicExch(a.status, 1); return; }
    const int nsp = n_splits_of(ctx, a.split_keys);
    if (split >= nsp) return;
    const int k_begin = split * a.split_keys;
    const int k_end = min(ctx, k_begin + a.split_keys);
    const bool last = split == nsp - 1;
    const int ctx_tiles = (k_end - k_begin + TK - 1) / TK;
    const int ntiles = ctx_tiles + (last ? 1 : 0);

    const uint32_t sQ = smem_u32(smem);
    const uint32_t sKV = sQ + 16 * ROWB;
    const int* table = a.block_table + (size_t)b * a.max_pages;

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
                    const int page = table[key / a.page_size];
                    if (page >= 0 && page < a.n_pages) off = (((long long)page * ATT_KV + kvh) * a.page_size + key % a.page_size) * ATT_D;
                }
            } else if (tid < M) {
                off = -2 - ((((long long)b * M + tid) * ATT_KV + kvh) * ATT_D);          // new rows live in k_new / v_new
            }
            row_off[stage * TK + tid] = off;
        }
    };
    auto load_tile = [&](int stage) {
        const uint32_t dK = sKV + stage * 2 * TILE_BYTES, dV = dK + TILE_BYTES;
        const int c = tid & 31;
#pragma unroll 4
        for (int i = 0; i < 8; i++) {
            const int r = (tid >> 5) + 8 * i;
            const long long off = row_off[stage * TK + r];
            const __nv_bfloat16 *srcK = a.k_pages, *srcV = a.v_pages;
            int bytes = 0;
            if (off >= 0) { srcK = a.k_pages + off; srcV = a.v_pages + off; bytes = 16; }
            else if (off <= -2) { srcK = a.k_new + (-2 - off); srcV = a.v_new + (-2 - off); bytes = 16; }
            cp_async16(dK + swz(r, c), reinterpret_cast<const uint4*>(srcK) + (bytes ? c : 0), bytes);
            cp_async16(dV + swz(r, c), reinterpret_cast<const uint4*>(srcV) + (bytes ? c : 0), bytes);
        }
    };

    float o[32][4];
#pragma unroll
    for (int n = 0; n < 32; n++) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float sc = 0.0625f * 1.4426950408889634f;          // 256^-1/2 (qwen35/batch.py:176), scores kept in log2 units

    // prologue: plan the first three tiles, start the first two
    for (int t = 0; t < ATT_STAGES && t < ntiles; t++) plan_tile(t, t);
    __syncthreads();
    for (int t = 0; t < ATT_STAGES - 1; t++) {
        if (t < ntiles) load_tile(t);
        cp_async_commit();
    }
    for (int t = 0; t < ntiles; t++) {
        const int stage = t % ATT_STAGES;
        // tile t+2 goes into the stage that tile t-1 used (all warps left it at the barrier that ended iteration t-1)
        if (t + ATT_STAGES - 1 < ntiles) load_tile((t + ATT_STAGES - 1) % ATT_STAGES);
        cp_async_commit();
        cp_async_wait<ATT_STAGES - 1>();
        __syncthreads();

        const bool new_tile = t >= ctx_tiles;
        const int key0 = new_tile ? 0 : k_begin + t * TK;               // position of the tile's first key in its own numbering
        const int limit = new_tile ? M : k_end - key0;                   // keys of the tile that exist
        if (warp * KPW < limit) {
            const uint32_t tK = sKV + stage * 2 * TILE_BYTES, tV = tK + TILE_BYTES;
            // scores of this warp's 8 keys: two accumulators (even / odd 16-wide slices of the head dim) halve the MMA chain
            float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int k2 = 0; k2 < 8; k2++) {
                uint32_t a0[4], a1[4], bfr[4];
                ldsm_x4(tK + swz(warp * KPW + (lane & 7), 4 * k2 + (lane >> 3)), bfr);
                ldsm_x4(sQ + swz((lane & 7) + 8 * ((lane >> 3) & 1), 4 * k2 + (lane >> 4)), a0);
                ldsm_x4(sQ + swz((lane & 7) + 8 * ((lane >> 3) & 1), 4 * k2 + 2 + (lane >> 4)), a1);
                mma_bf16(s0, a0, bfr[0], bfr[1]);
                mma_bf16(s1, a1, bfr[2], bfr[3]);
            }
            // mask + online softmax; thread holds rows g (e = 0,1) and g + 8 (e = 2,3), keys 8*warp + 2*t4 + (e & 1)
            float sv[4], mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int kk = warp * KPW + 2 * t4 + (e & 1);
                const int row = g + 8 * (e >> 1);
                const bool ok = new_tile ? (kk < M && kk <= (row >> 2)) : (kk < limit);
                sv[e] = ok ? (s0[e] + s1[e]) * sc : -INFINITY;
                mx[e >> 1] = fmaxf(mx[e >> 1], sv[e]);
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
            uint32_t pf[2], pl[2];
            {
                float p[4];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float mn = m_run[e >> 1];
                    p[e] = (mn == -INFINITY) ? 0.f : exp2f(sv[e] - mn);
                    l_run[e >> 1] += p[e];
                }
                pf[0] = pack_bf16x2(p[0], p[1]); pf[1] = pack_bf16x2(p[2], p[3]);
                // low parts: p - bf16(p), exact in fp32, then rounded to bf16 (16 significand bits in total)
#pragma unroll
                for (int e = 0; e < 4; e++) p[e] -= bf(p[e]);
                pl[0] = pack_bf16x2(p[0], p[1]); pl[1] = pack_bf16x2(p[2], p[3]);
            }
#pragma unroll
            for (int n = 0; n < 32; n++) { o[n][0] *= alpha[0]; o[n][1] *= alpha[0]; o[n][2] *= alpha[1]; o[n][3] *= alpha[1]; }
#pragma unroll
            for (int nq = 0; nq < 8; nq++) {
                uint32_t vf[4];
                ldsm_x4_t(tV + swz(warp * KPW + (lane & 7), 4 * nq + (lane >> 3)), vf);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    mma_bf16_k8(o[4 * nq + i], pf[0], pf[1], vf[i]);
                    mma_bf16_k8(o[4 * nq + i], pl[0], pl[1], vf[i]);
                }
            }
        }
        // this tile's row offsets were consumed two iterations ago: plan tile t+3 into the same slot; the barrier below orders
        // the plan before the load at the top of iteration t+1
        if (t + ATT_STAGES < ntiles) plan_tile(t + ATT_STAGES, stage);
        __syncthreads();
    }
    cp_async_wait<0>();
    __syncthreads();

    // ---- merge the four warps (each saw a different quarter of every tile) through shared memory ----
    float* mO = reinterpret_cast<float*>(smem + 16 * ROWB);              // [8][16][256]
    float* mML = mO + ATT_WARPS * 16 * ATT_D;                            // [8][16][2]
#pragma unroll
    for (int h = 0; h < 2; h++) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
#pragma unroll
    for (int n = 0; n < 32; n++) {
        float* p0 = mO + ((warp * 16 + g) * ATT_D) + 8 * n + 2 * t4;
        p0[0] = o[n][0]; p0[1] = o[n][1];
        p0[8 * ATT_D] = o[n][2]; p0[8 * ATT_D + 1] = o[n][3];
    }
    if (t4 == 0) {
        mML[(warp * 16 + g) * 2] = m_run[0]; mML[(warp * 16 + g) * 2 + 1] = l_run[0];
        mML[(warp * 16 + g + 8) * 2] = m_run[1]; mML[(warp * 16 + g + 8) * 2 + 1] = l_run[1];
    }
    __syncthreads();
    float* part = a.part + (((size_t)b * ATT_KV + kvh) * a.max_splits + split) * PART_STRIDE;
    for (int r = 0; r < 4 * M; r++) {
        float mw[ATT_WARPS], mstar = -INFINITY;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; w++) { mw[w] = mML[(w * 16 + r) * 2]; mstar = fmaxf(mstar, mw[w]); }
        float wgt[ATT_WARPS], lsum = 0.f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; w++) { wgt[w] = (mw[w] == -INFINITY) ? 0.f : exp2f(mw[w] - mstar); lsum += wgt[w] * mML[(w * 16 + r) * 2 + 1]; }
        {
            const int d = tid;                                           // 256 threads = 256 dims
            float acc = 0.f;
#pragma unroll
            for (int w = 0; w < ATT_WARPS; w++) acc += wgt[w] * mO[(w * 16 + r) * ATT_D + d];
            part[r * ATT_D + d] = acc;
        }
        if (tid == 0) { part[16 * ATT_D + 2 * r] = mstar; part[16 * ATT_D + 2 * r + 1] = lsum; }
    }
}

// merge the splits of one (row, query head): 128 threads x 2 dims
__global__ void __launch_bounds__(128) gqa_decode_merge_kernel(const AttnArgs a) {
    const int r = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int b = r / a.M, j = r % a.M, kvh = h / ATT_GQA, row = j * 4 + (h % ATT_GQA);
    const int ctx = a.ctx_len[b];
    if (ctx < 0 || (long long)ctx + a.M > (long long)a.max_pages * a.page_size) return;
    const int nsp = n_splits_of(ctx, a.split_keys);
    const float* base = a.part + ((size_t)b * ATT_KV + kvh) * a.max_splits * PART_STRIDE;
    float mstar = -INFINITY;
    for (int s = 0; s < nsp; s++) mstar = fmaxf(mstar, base[(size_t)s * PART_STRIDE + 16 * ATT_D + 2 * row]);
    float acc0 = 0.f, acc1 = 0.f, lsum = 0.f;
    for (int s = 0; s < nsp; s++) {
        const float* p = base + (size_t)s * PART_STRIDE;
        const float m = p[16 * ATT_D + 2 * row];
        const float w = (m == -INFINITY) ? 0.f : exp2f(m - mstar);
        lsum += w * p[16 * ATT_D + 2 * row + 1];
        acc0 += w * p[row * ATT_D + tid];
        acc1 += w * p[row * ATT_D + tid + 128];
    }
    const float inv = lsum == 0.f ? 1.f : 1.f / lsum;                  // sum == 0 guard as qwen35/batch.py:216
    __nv_bfloat16* o = a.out + ((size_t)r * ATT_H + h) * ATT_D;
    o[tid] = __float2bfloat16_rn(acc0 * inv);
    o[tid + 128] = __float2bfloat16_rn(acc1 * inv);
}

// split size (keys): a block has a fixed cost (pipeline fill, the merge of its eight warps, its partial) of several tile times, so
// splits are as long as they can be while a batch of B sequences of up to max_ctx keys still gives about one block per SM
void gqa_split_plan(int B, int max_ctx, int* split_keys, int* max_splits) {
    long long sk = (long long)max_ctx * B * ATT_KV / 200;
    sk = (sk / TK) * TK;
    if (sk < 2 * TK) sk = 2 * TK;
    if (sk > 4096) sk = 4096;
    int ms = (int)((max_ctx + sk - 1) / sk);
    if (ms < 1) ms = 1;
    *split_keys = (int)sk;
    *max_splits = ms;
}

size_t gqa_workspace_bytes(int B, int max_ctx) {
    int sk, ms;
    gqa_split_plan(B, max_ctx, &sk, &ms);
    return (size_t)B * ATT_KV * ms * PART_STRIDE * sizeof(float);
}

int launch_gqa_decode(AttnArgs a, int max_ctx, cudaStream_t stream) {
    if (a.B <= 0) return GDN_OK;
    gqa_split_plan(a.B, max_ctx, &a.split_keys, &a.max_splits);
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !attr_set[dev]) {
        if (cudaFuncSetAttribute(gqa_decode_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM) != cudaSuccess)
            return check_launch("gqa_decode smem attribute");
        attr_set[dev] = true;
    }
    gqa_decode_split_kernel<<<dim3(a.max_splits, ATT_KV, a.B), ATT_THREADS, ATT_SMEM, stream>>>(a);
    int rc = check_launch("gqa_decode_split");
    if (rc) return rc;
    gqa_decode_merge_kernel<<<dim3(a.B * a.M, ATT_H), 128, 0, stream>>>(a);
    return check_launch("gqa_decode_merge");
}

// ----------------------------------------------------------------------------------------------------------------------
// Variant for callers that cannot allocate device memory: the split-KV partials go to a fixed array that lives in the library
// image instead of a caller-provided workspace.  Every GPU that loads the library holds these 12 MiB until the process exits.
// The array is shared by all calls on a device and keeps whatever the last call left in it; nothing in it has to start at zero
// (every partial that the merge kernel reads was written by the split kernel of the same call), but two calls that overlap on
// the GPU (different streams) would overwrite each other's partials.
// ----------------------------------------------------------------------------------------------------------------------
constexpr int STATIC_PARTIALS = 762;                                   // (sequence, kv head, split) triples that fit
static __device__ __align__(256) float g_static_partials[(size_t)STATIC_PARTIALS * PART_STRIDE];      // 12 MiB

int gqa_static_max_partials() { return STATIC_PARTIALS; }

int launch_gqa_decode_static(AttnArgs a, int max_ctx, cudaStream_t stream) {
    if (a.B <= 0) return GDN_OK;
    int sk, ms;
    gqa_split_plan(a.B, max_ctx, &sk, &ms);
    const long long need = (long long)a.B * ATT_KV * ms;
    if (need > STATIC_PARTIALS) {
        set_error("gqa_decode_paged_static: B=%d sequences of up to %d tokens need %lld split partials, the built-in scratch holds %d "
                  "(use gqa_decode_paged with a workspace of gqa_decode_workspace_bytes() instead)", a.B, max_ctx, need, STATIC_PARTIALS);
        return GDN_E_SHAPE;
    }
    // In host code the array's name is only a handle: the device address has to be asked for, once per device, with that device
    // current.  The first call on a device does it (and should therefore come before any stream capture).
    static float* addr[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return check_launch("gqa_decode_paged_static: device");
    if (!addr[dev]) {
        float* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_partials);
        if (e != cudaSuccess || !p) {
            cudaGetLastError();
            set_error("gqa_decode_paged_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return GDN_E_LAUNCH;
        }
        addr[dev] = p;
    }
    a.part = addr[dev];
    return launch_gqa_decode(a, max_ctx, stream);
}

}  // namespace gdn
