// Causal prefill attention, head_dim 256, GQA 8 query heads on 2 KV heads, on the Blackwell tensor cores (tcgen05 / TMEM / TMA).
//
// Replaces the scaled-dot-product call of the reference's prefill (qwen35/model.py:148-169, the `mx.fast.scaled_dot_product_attention`
// at :165, reached from qwen35/prefill.py:468): for the S query tokens at positions pos .. pos + S - 1,
//     o[i, h, :] = softmax(q[i, h, :] . K[0 .. pos + i, h / 4, :] / 16) V[0 .. pos + i, h / 4, :]
// with bf16 inputs and output and fp32 scores, sums and accumulation.
//
// One block per (KV head, 32 query tokens): the 4 query heads that share the KV head and the 32 tokens make the 128 rows of the
// tensor-core tile (row = token * 4 + head), so a K / V tile is read once for four heads.  Per 64-key tile:
//     S [128 x 64]   = Q K^T        16 MMAs (K = 256 dims), A = Q (shared memory, loaded once), B = the K tile as TMA wrote it
//     P              = 2^(S sc - m) one thread per row (no cross-lane reduction), bf16 hi + lo pairs into tensor memory
//     O [128 x 256] += P V          8 MMAs (K = 64 keys, hi and lo), A = P from tensor memory, B = the V tile read N-major
// S and P are double buffered in tensor memory (O 256 + 2 x 64 + 2 x 64 columns = 512): the softmax of tile t runs while the tensor
// pipe forms the scores of tile t + 1.  The running maximum is only raised when a tile exceeds it by more than 2^8, so the rescale
// of O (a round trip through registers) is rare; l and O carry the same reference, so the result does not depend on it.
// Blocks are numbered so that the ones with the most keys (the last query tokens) start first.
//
// Roles (192 threads): warps 0-3 softmax / epilogue (thread = row = TMEM lane), warp 4 lane 0 issues the MMAs, warp 5 lane 0 is the
// TMA producer (Q once, then two-stage rings of K and of V tiles, each with its own barriers).  Every wait is bounded; a wait that gives up sets the device status
// word and the block runs out its loops without touching the tensor cores again.
#include <cuda.h>
#include <cstring>
#include "gqa_common.cuh"
#include "sm100_prims.cuh"

namespace gdn {

using namespace sm100;

constexpr int PF_THREADS = 192;
constexpr int PF_QTOK = 32;                                          // query tokens per block (x 4 heads = 128 rows)
constexpr int PF_STAGES = 2;
constexpr int PF_Q_BYTES = 128 * ATT_D * 2;                          // 64 KiB: 4 slabs of [128 rows][64 dims]
constexpr int PF_SMEM = PF_Q_BYTES + PF_STAGES * 2 * TILE_BYTES;     // + two stages of K + V tiles (192 KiB)
constexpr uint32_t PFM_O = 0, PFM_S0 = 256, PFM_P0 = 384;            // O [256], S buffers [64] x 2, P buffers [hi 32 | lo 32] x 2
enum { PB_QFULL = 0, PB_KFULL0 = 1, PB_KEMPTY0 = 3, PB_VFULL0 = 5, PB_VEMPTY0 = 7, PB_SDONE0 = 9, PB_SFREE0 = 11, PB_PREADY0 = 13, PB_PFREE0 = 15,
       PB_ODONE = 17, PB_COUNT = 18 };
constexpr float PF_RESCALE_STEP = 8.f;                               // log2 units

struct PrefillAttnArgs {
    __nv_bfloat16* out;        // [S, 8, 256]
    int S, pos;                // query tokens and the position of the first one; keys 0 .. pos + S - 1 exist
    int kv_head_major;         // K / V are [2, T, 256] (the tensor maps then order their dimensions (256, T, 2)) instead of [T, 2, 256]
    int* status;
};

__global__ void __launch_bounds__(PF_THREADS, 1)
gqa_prefill_tc_kernel(const PrefillAttnArgs a, const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV) {
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ uint64_t bars[PB_COUNT];
    __shared__ uint32_t tmem_slot;
    __shared__ int s_abort;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t sbase = smem_addr(smem);
    if (sbase & 1023u) { if (tid == 0) atomicExch(a.status, 4); return; }
    const int n_qb = (a.S + PF_QTOK - 1) / PF_QTOK;
    const int qb = n_qb - 1 - (int)(blockIdx.x >> 1), kvh = (int)(blockIdx.x & 1);     // most keys first
    const int tok0 = qb * PF_QTOK;                                   // first query token of the block (relative to the call)
    const int last_key = a.pos + min(tok0 + PF_QTOK, a.S) - 1;       // the last key any row of the block sees
    const int ntiles = last_key / TK + 1;

    auto bar = [&](int i) -> uint32_t { return smem_addr(&bars[i]); };
    if (tid == 0) {
        mbar_init(bar(PB_QFULL), 1);
        for (int i = 0; i < 2; i++) {
            mbar_init(bar(PB_KFULL0 + i), 1); mbar_init(bar(PB_KEMPTY0 + i), 1);
            mbar_init(bar(PB_VFULL0 + i), 1); mbar_init(bar(PB_VEMPTY0 + i), 1);
            mbar_init(bar(PB_SDONE0 + i), 1); mbar_init(bar(PB_SFREE0 + i), 4);
            mbar_init(bar(PB_PREADY0 + i), 4); mbar_init(bar(PB_PFREE0 + i), 1);
        }
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
    const uint32_t sQ = sbase, sKV = sbase + PF_Q_BYTES;

    if (warp == 5) {
        // ================= producer =================
        if (lane == 0) {
            mbar_expect_tx(bar(PB_QFULL), PF_Q_BYTES);
            for (int j = 0; j < 4; j++) tma_load_3d(sQ + j * 16384, &tmQ, bar(PB_QFULL), 64 * j, kvh * ATT_GQA, tok0);
            // K and V tiles have their own barriers: the K buffer of a stage is free as soon as the scores of its tile are formed, the
            // V buffer when the tile's P V product is done; the copies are issued in the order in which the buffers come free
            // (K of tile n + 1 before V of tile n), each a whole tile ahead of its use
            auto load_k = [&](int n) -> bool {
                const int stage = n % PF_STAGES;
                if (n >= PF_STAGES && !wait(PB_KEMPTY0 + stage, (uint32_t)(n / PF_STAGES) - 1)) return false;
                const uint32_t dK = sKV + stage * 2 * TILE_BYTES;
                mbar_expect_tx(bar(PB_KFULL0 + stage), TILE_BYTES);
                for (int j = 0; j < 4; j++)
                    tma_load_3d(dK + j * 8192, &tmK, bar(PB_KFULL0 + stage), 64 * j, a.kv_head_major ? n * TK : kvh, a.kv_head_major ? kvh : n * TK);
                return true;
            };
            auto load_v = [&](int n) -> bool {
                const int stage = n % PF_STAGES;
                if (n >= PF_STAGES && !wait(PB_VEMPTY0 + stage, (uint32_t)(n / PF_STAGES) - 1)) return false;
                const uint32_t dV = sKV + stage * 2 * TILE_BYTES + TILE_BYTES;
                mbar_expect_tx(bar(PB_VFULL0 + stage), TILE_BYTES);
                for (int j = 0; j < 4; j++)
                    tma_load_3d(dV + j * 8192, &tmV, bar(PB_VFULL0 + stage), 64 * j, a.kv_head_major ? n * TK : kvh, a.kv_head_major ? kvh : n * TK);
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
            constexpr uint32_t I_QK = idesc_bf16(128, 64, 0, 0);
            constexpr uint32_t I_PV = idesc_bf16(128, 256, 0, 1);    // B = V read N-major (dims contiguous)
            constexpr uint32_t HI = smem_desc_hi_sw128(1024);
            auto issue_pv = [&](int m) -> bool {
                const int buf = m & 1, stage = m % PF_STAGES;
                if (!wait(PB_PREADY0 + buf, (uint32_t)(m >> 1)) || !wait(PB_VFULL0 + stage, (uint32_t)(m / PF_STAGES))) return false;
                tc_fence_after_sync();
                const uint32_t vlo = smem_desc_lo(sKV + stage * 2 * TILE_BYTES + TILE_BYTES, 8192);
                for (int part = 0; part < 2; part++)
                    for (int ks = 0; ks < 4; ks++) {
                        const uint32_t acol = tb + PFM_P0 + buf * 64 + part * 32 + ks * 8;
                        if (m == 0 && part == 0 && ks == 0) mma_ts_w<false>(tb + PFM_O, acol, vlo + ks * 128, HI, I_PV);
                        else mma_ts_w<true>(tb + PFM_O, acol, vlo + ks * 128, HI, I_PV);
                    }
                mma_commit(bar(PB_VEMPTY0 + stage));
                mma_commit(bar(PB_PFREE0 + buf));
                return true;
            };
            bool ok = wait(PB_QFULL, 0);
            tc_fence_after_sync();
            const uint32_t qlo = smem_desc_lo(sQ, 16);
            for (int n = 0; n < ntiles && ok && !aborted(); n++) {
                const int buf = n & 1, stage = n % PF_STAGES;
                ok = wait(PB_KFULL0 + stage, (uint32_t)(n / PF_STAGES)) && (n < 2 || wait(PB_SFREE0 + buf, (uint32_t)(n >> 1) - 1));
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t klo = smem_desc_lo(sKV + stage * 2 * TILE_BYTES, 16);
#pragma unroll
                for (int ks = 0; ks < 16; ks++) {
                    const uint32_t qo = (ks >> 2) * (16384 >> 4) + (ks & 3) * 2, ko = (ks >> 2) * (8192 >> 4) + (ks & 3) * 2;
                    if (ks == 0) mma_ss_w<false>(tb + PFM_S0 + buf * 64, qlo + qo, HI, klo + ko, HI, I_QK);
                    else mma_ss_w<true>(tb + PFM_S0 + buf * 64, qlo + qo, HI, klo + ko, HI, I_QK);
                }
                mma_commit(bar(PB_KEMPTY0 + stage));
                mma_commit(bar(PB_SDONE0 + buf));
                if (n >= 1) ok = issue_pv(n - 1);
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
            const int buf = n & 1;
            if (!wait(PB_SDONE0 + buf, (uint32_t)(n >> 1))) { ok = false; break; }
            tc_fence_after_sync();
            float s[64];
            {
                uint32_t r0[32], r1[32];
                tmem_ld32(tl + PFM_S0 + buf * 64, r0);
                tmem_ld32(tl + PFM_S0 + buf * 64 + 32, r1);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; i++) { s[i] = __uint_as_float(r0[i]); s[32 + i] = __uint_as_float(r1[i]); }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(PB_SFREE0 + buf));        // the score columns may take tile n + 2
            if (n * TK + TK - 1 > a.pos + tok0) {                    // the tile reaches past the block's first query: causal mask
#pragma unroll
                for (int i = 0; i < 64; i++) s[i] = (n * TK + i <= my_pos) ? s[i] : -INFINITY;
            }
            float mt = -INFINITY;
#pragma unroll
            for (int i = 0; i < 64; i++) mt = fmaxf(mt, s[i]);
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
            // p = 2^(s sc - m); a masked score (-inf) gives 0
            uint32_t ph[32], pl[32];
            const float nm = (m_run == -INFINITY) ? 0.f : -m_run;
#pragma unroll
            for (int i = 0; i < 64; i += 2) {
                float p0, p1;
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p0) : "f"(fmaf(s[i], sc, nm)));
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p1) : "f"(fmaf(s[i + 1], sc, nm)));
                l_run += p0 + p1;
                ph[i >> 1] = pack_bf16x2(p0, p1);
                pl[i >> 1] = pack_bf16x2(p0 - __uint_as_float(ph[i >> 1] << 16), p1 - __uint_as_float(ph[i >> 1] & 0xffff0000u));
            }
            if (n >= 2 && !wait(PB_PFREE0 + buf, (uint32_t)(n >> 1) - 1)) { ok = false; break; }      // P V of tile n - 2 has read this buffer
            tc_fence_after_sync();
            tmem_st32(tl + PFM_P0 + buf * 64, ph);
            tmem_st32(tl + PFM_P0 + buf * 64 + 32, pl);
            tmem_wait_st();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(PB_PREADY0 + buf));
        }
        // ---- epilogue: o = O / l ----
        if (ok) ok = wait(PB_ODONE, 0);
        tc_fence_after_sync();
        const float inv = l_run == 0.f ? 1.f : 1.f / l_run;
        const bool row_ok = ok && tok < a.S;
        __nv_bfloat16* orow = a.out + ((size_t)tok * ATT_H + kvh * ATT_GQA + (row & 3)) * ATT_D;
#pragma unroll 1
        for (int c0 = 0; c0 < 256; c0 += 32) {
            uint32_t o[32];
            tmem_ld32(tl + PFM_O + c0, o);
            tmem_wait_ld();
            if (row_ok) {
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    uint4 v;
                    v.x = pack_bf16x2(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
                    v.y = pack_bf16x2(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
                    v.z = pack_bf16x2(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
                    v.w = pack_bf16x2(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
                    *reinterpret_cast<uint4*>(orow + c0 + i) = v;
                }
            }
        }
        tc_fence_before_sync();
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 4) tmem_dealloc(tb, 512);
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

int launch_gqa_prefill(const void* q, const void* k, const void* v, void* out, int S, int pos, long long k_tok_stride, long long k_head_stride,
                       long long v_tok_stride, long long v_head_stride, int* status, cudaStream_t stream) {
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
    if (head_major) okm = okm && make_map3(&tk, k, T, ATT_KV, k_tok_stride, k_head_stride, TK, 1) && make_map3(&tv, v, T, ATT_KV, v_tok_stride, v_head_stride, TK, 1);
    else okm = okm && make_map3(&tk, k, ATT_KV, T, k_head_stride, k_tok_stride, 1, TK) && make_map3(&tv, v, ATT_KV, T, v_head_stride, v_tok_stride, 1, TK);
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
    gqa_prefill_tc_kernel<<<n_qb * ATT_KV, PF_THREADS, PF_SMEM, stream>>>(a, tq, tk, tv);
    return check_launch("gqa_prefill_attn");
}

}  // namespace gdn
