// GatedDeltaNet recurrent decode / speculative-verify kernel.
//
// One launch runs M chained tokens for each of B sequences: depthwise causal conv (4 taps) + silu on the mixed qkv row,
// q/k l2norm, gates, the gated delta rule on the fp32 [16,128,128] state, and a state + conv-window snapshot after every
// token.  It replaces three Metal kernels of the reference that share this arithmetic and differ only in where the state
// lives: `deltanet` (qwen35/kernels.py:461-567, functional snapshots), `deltanet_b` (qwen35/batch.py:36-135, slot pools
// updated in place) and `deltanet_bm` (qwen35/batch_spec.py:45-150, snapshot pools updated in place).
//
// The kernel is bound by HBM traffic on the state (1 MiB read + M MiB written per sequence and layer), so it is built as
// a streaming pipeline:
//   * the work list is every 32-row slice (16 KiB) of every (sequence, head) state; persistent blocks (three or four per SM) each take
//     a contiguous range of it, so consecutive slices of a block usually belong to the same head;
//   * a ring of shared-memory stages per block is kept full by one thread issuing 16 KiB bulk async copies (cp.async.bulk,
//     completion on an mbarrier), so ~190 KiB of state reads are in flight per SM regardless of what the math is doing;
//   * a slice is moved from shared memory to registers (a state row = 8 lanes x 4 float4, so each quarter-warp reads 128
//     contiguous bytes), the stage is handed back to the copy engine, the M tokens are applied in registers and each snapshot
//     is streamed out with 128-bit stores; the two 128-wide dot products per row end in three xor-shuffles;
//   * the conv / l2norm / gate prologue of a head is computed once per head into shared memory (thread t = channel t of
//     q, k and v) from inputs that were fetched into registers while the previous head was being processed.
#include "gdn_common.cuh"
#include "launchers.cuh"
#include "sm100_prims.cuh"

namespace gdn {

constexpr int SLICE_ROWS = 32;
constexpr int SLICES_PER_HEAD = DV / SLICE_ROWS;             // 4
constexpr int SLICE_FLOATS = SLICE_ROWS * DK;                // 4096
constexpr int SLICE_BYTES = SLICE_FLOATS * 4;                // 16 KiB
// ring stages and resident blocks per SM, by the number of chained tokens a block keeps inputs for: the single-token decode
// step needs many warps to cover the latency of its shuffle / FMA chains (4 blocks x 3 stages = 192 KiB of reads in flight per
// SM); the multi-token verify is write-dominated and register-heavy (3 blocks x 4 stages)
template <int MT> struct Tune { static constexpr int NST = MT == 1 ? 3 : 4; static constexpr int BLOCKS = MT == 1 ? 4 : (MT <= 4 ? 3 : 2); };

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// where one sequence's state and conv window live (qwen35/kernels.py:473-474, batch.py:47-54, batch_spec.py:57-65)
struct SeqPtrs {
    const __nv_bfloat16* cs_in;
    __nv_bfloat16* cs_out;
    const float* st_in;
    float* st_out;
    bool ok;
};

// the index words of sequence b, as loaded (the loads are independent of one another: issuing them costs nothing until a value is used)
struct RawIdx { int e, i1, i2; };
__device__ __forceinline__ RawIdx load_idx(const DecodeArgs& a, int b) {
    RawIdx r;
    r.e = a.i0[a.mode == 0 ? 0 : b];
    r.i1 = a.mode == 0 ? 0 : a.i1[b];
    r.i2 = a.mode == 2 ? a.i2[b] : 0;
    return r;
}

__device__ __forceinline__ SeqPtrs make_ptrs(const DecodeArgs& a, const RawIdx& r) {
    SeqPtrs p;
    const int M = a.M;
    const int e = r.e;
    p.ok = e >= 0 && e < a.n_entries;
    const size_t es = p.ok ? (size_t)e : 0;
    if (a.mode == 0) {
        p.cs_in = a.conv_pool + es * 3 * CD;
        p.cs_out = a.conv_out;
        p.st_in = a.ssm_pool + es * STATE_ELEMS;
        p.st_out = a.ssm_out;
    } else if (a.mode == 1) {
        const unsigned par = (unsigned)r.i1 & 1u;
        p.cs_in = a.conv_pool + (es * 2 + par) * 3 * CD;
        p.cs_out = a.conv_pool + (es * 2 + (par ^ 1u)) * 3 * CD;
        p.st_in = a.ssm_pool + es * STATE_ELEMS;
        p.st_out = a.ssm_pool + es * STATE_ELEMS;
    } else {
        int sl = r.i1;
        if (sl < 0 || sl >= M) { p.ok = false; sl = 0; }
        const unsigned par = (unsigned)r.i2 & 1u;
        p.cs_in = a.conv_pool + ((es * 2 + par) * M + sl) * 3 * CD;
        p.cs_out = a.conv_pool + ((es * 2 + (par ^ 1u)) * M) * 3 * CD;
        p.st_out = a.ssm_pool + es * M * STATE_ELEMS;
        p.st_in = p.st_out + (size_t)sl * STATE_ELEMS;
    }
    return p;
}
__device__ __forceinline__ SeqPtrs resolve(const DecodeArgs& a, int b) { return make_ptrs(a, load_idx(a, b)); }

// raw inputs of one thread's three channels (q, k, v channel `tid` of a head) for MT chained tokens
// (kept as raw bf16 bits: converting at the point of use keeps the loads asynchronous when they are issued one head ahead)
template <int MT>
struct HeadInputs {
    unsigned short win[3][3];    // stored window rows (t = -3, -2, -1)
    unsigned short row[3][MT];   // new rows (t = 0 .. M-1)
    uint2 w[3];                  // conv taps (4 bf16)
    unsigned short a[MT], b[MT]; // gate inputs of the head
};
__device__ __forceinline__ unsigned short ldraw(const __nv_bfloat16* p) { return *reinterpret_cast<const unsigned short*>(p); }
__device__ __forceinline__ float rawf(unsigned short u) { return __uint_as_float((uint32_t)u << 16); }

template <int MT>
__device__ __forceinline__ void fetch_head(const DecodeArgs& a, const SeqPtrs& sp, int b, int hv, int tid, HeadInputs<MT>& in) {
    const __nv_bfloat16* pj = a.proj + (size_t)b * a.M * a.row_stride;
#pragma unroll
    for (int g = 0; g < 3; g++) {
        const int ch = g * KD + hv * DK + tid;
        in.w[g] = *reinterpret_cast<const uint2*>(a.conv_w + (size_t)ch * 4);
#pragma unroll
        for (int t = 0; t < 3; t++) in.win[g][t] = ldraw(sp.cs_in + t * CD + ch);
#pragma unroll
        for (int j = 0; j < MT; j++) in.row[g][j] = j < a.M ? ldraw(pj + (size_t)j * a.row_stride + ch) : (unsigned short)0;
    }
#pragma unroll
    for (int j = 0; j < MT; j++) {
        in.a[j] = j < a.M ? ldraw(pj + (size_t)j * a.row_stride + CD + KD + HV + hv) : (unsigned short)0;
        in.b[j] = j < a.M ? ldraw(pj + (size_t)j * a.row_stride + CD + KD + hv) : (unsigned short)0;
    }
}

template <int MT>
__global__ void __launch_bounds__(128, Tune<MT>::BLOCKS) gdn_decode_kernel(const DecodeArgs a, int n_slices) {
    constexpr int NST = Tune<MT>::NST;
    extern __shared__ __align__(128) unsigned char dsmem[];
    float* ring = reinterpret_cast<float*>(dsmem);                                  // [NST][SLICE_FLOATS]
    float* sq = ring + NST * SLICE_FLOATS;                                          // [MT][128]
    float* sk = sq + MT * DK;
    float* sv = sk + MT * DK;
    float* sred = sv + MT * DV;                                                     // [2*MT][4]
    float* sgate = sred + 2 * MT * 4;                                               // [MT][2] (g, beta)
    __shared__ uint64_t full_bar[NST];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, sub = lane >> 3, l8 = lane & 7;
    const int M = a.M;
    const int G = gridDim.x;
    const int lo = (int)((long long)blockIdx.x * n_slices / G), hi = (int)((long long)(blockIdx.x + 1) * n_slices / G);
    // Programmatic dependent launch: the next kernel of the stream may be scheduled onto SMs as this one leaves them; this one waits
    // here, before it reads anything an earlier kernel may have written, until its predecessors have completed.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (lo >= hi) return;

    if (tid == 0) {
        for (int s = 0; s < NST; s++) sm100::mbar_init(sm100::smem_addr(&full_bar[s]), 1);
        sm100::fence_barrier_init();
    }
    __syncthreads();

    // thread 0: start the copy of slice `idx` into its ring stage; st_in = the state of the slice's sequence
    auto issue = [&](int idx, const float* st_in) {
        const int n = idx - lo, stage = n % NST;
        const int hv = (idx / SLICES_PER_HEAD) % HV, sl = idx % SLICES_PER_HEAD;
        const float* src = st_in + ((size_t)hv * DV + sl * SLICE_ROWS) * DK;
        const uint32_t bar = sm100::smem_addr(&full_bar[stage]);
        sm100::mbar_expect_tx(bar, SLICE_BYTES);
        bulk_load(sm100::smem_addr(ring + stage * SLICE_FLOATS), src, SLICE_BYTES, bar);
    };

    const float inv_scale = 0.08838834764831845f;          // 128^-1/2
    const float e2 = 1e-6f * inv_scale * inv_scale;
    const float sc_q = bf(inv_scale * inv_scale), sc_k = bf(inv_scale);

    GDN_BSTAMP(0);
    // Everything a head's prologue needs -- the sequence's pointers included -- is fetched into registers one head ahead (`nxt*`):
    // a load issued while the bulk copies saturate the memory system takes microseconds (measured: 3.5 us for the first index word
    // when it was issued behind the ring's copies, and 3 us per further head of a block for the same word), so neither the prologue
    // nor the thread that refills the ring may wait for one.  For the first head the loads go out before the ring's copies.
    // (Loading the index words two heads ahead, so that the prefetch itself never waits for them, measured 1.5% slower.)
    HeadInputs<MT> nxt;
    SeqPtrs nxt_sp{};
    float nxt_alog = 0.f, nxt_dtb = 0.f;
    int have_b = -1, have_hv = -1;                         // head whose inputs sit in `nxt`
    int cur_b = -1, cur_hv = -1;
    SeqPtrs sp{};
    auto prefetch_head = [&](int pb, int phv) {
        nxt_sp = resolve(a, pb);
        fetch_head<MT>(a, nxt_sp, pb, phv, tid, nxt);
        nxt_alog = a.A_log[phv];
        nxt_dtb = a.dt_bias[phv];
        have_b = pb; have_hv = phv;
    };
    prefetch_head(lo / (HV * SLICES_PER_HEAD), (lo / SLICES_PER_HEAD) % HV);
    if (tid == 0)
        for (int i = lo; i < hi && i < lo + NST; i++) {
            const int ib = i / (HV * SLICES_PER_HEAD);
            issue(i, ib == have_b ? nxt_sp.st_in : resolve(a, ib).st_in);
        }

    for (int idx = lo; idx < hi; idx++) {
        const int n = idx - lo, stage = n % NST;
        const int b = idx / (HV * SLICES_PER_HEAD), hv = (idx / SLICES_PER_HEAD) % HV, sl = idx % SLICES_PER_HEAD;

        if (b != cur_b || hv != cur_hv) {
            // ---- prologue of a new head: conv + silu, l2norm, gates for the M tokens, conv-window snapshots ----
            cur_b = b; cur_hv = hv;
            if (have_b != b || have_hv != hv) prefetch_head(b, hv);      // (does not happen: every head is fetched one head ahead)
            sp = nxt_sp;
            const HeadInputs<MT> in = nxt;
            const float alog = nxt_alog, dtb = nxt_dtb;
            if (!sp.ok && tid == 0) atomicExch(a.status, 1);
            if (idx == lo) GDN_BSTAMP(10);
            // start fetching the next head of this block's range while this one is processed
            {
                const int nidx = (idx / SLICES_PER_HEAD + 1) * SLICES_PER_HEAD;
                if (nidx < hi) prefetch_head(nidx / (HV * SLICES_PER_HEAD), (nidx / SLICES_PER_HEAD) % HV);
            }
            __syncthreads();                               // previous head's readers of sq/sk/sv are done
            if (idx == lo) GDN_BSTAMP(11);
            float qv[MT], kv[MT];
            const float expA = expf(alog);
#pragma unroll
            for (int j = 0; j < MT; j++) {
                if (j < M) {
                    float c[3];
#pragma unroll
                    for (int g = 0; g < 3; g++) {
                        // input rows j-3 .. j of the channel: the stored window for t < 0, the new rows otherwise (kernels.py:477-484)
                        float x[4], w[4];
                        unpack_bf16x4(in.w[g], w);
#pragma unroll
                        for (int t = 0; t < 4; t++) {
                            const int tt = j - 3 + t;
                            x[t] = rawf(tt < 0 ? in.win[g][tt + 3] : in.row[g][tt < 0 ? 0 : tt]);
                        }
                        float o = x[0] * w[0];
                        o += x[1] * w[1];
                        o += x[2] * w[2];
                        o += x[3] * w[3];
                        c[g] = silu_bf16(bf(o));
                    }
                    qv[j] = c[0]; kv[j] = c[1];
                    sv[j * DV + tid] = c[2];
                    const float qs_w = warp_sum(c[0] * c[0]), ks_w = warp_sum(c[1] * c[1]);
                    if (lane == 0) { sred[(2 * j) * 4 + warp] = qs_w; sred[(2 * j + 1) * 4 + warp] = ks_w; }
                    // the gates of the chained tokens on different warps (decay on one, beta on another): side by side, not in a row
                    if (tid == 32 * (j & 3)) sgate[2 * j] = expf(log_decay(expA, rawf(in.a[j]), dtb));
                    if (tid == 32 * ((j + 2) & 3)) sgate[2 * j + 1] = sigmoid_bf16(rawf(in.b[j]));
                    // conv-window snapshot j = input rows j-2, j-1, j (kernels.py:528-541); written by the block that owns slice 0
                    if (sl == 0 && sp.ok) {
#pragma unroll
                        for (int g = 0; g < 3; g++) {
                            const int ch = g * KD + hv * DK + tid;
#pragma unroll
                            for (int t = 0; t < 3; t++) {
                                const int tt = j - 2 + t;
                                const unsigned short x = tt < 0 ? in.win[g][tt + 3] : in.row[g][tt < 0 ? 0 : tt];
                                *reinterpret_cast<unsigned short*>(sp.cs_out + ((size_t)j * 3 + t) * CD + ch) = x;
                            }
                        }
                    }
                }
            }
            __syncthreads();
#pragma unroll
            for (int j = 0; j < MT; j++) {
                if (j < M) {
                    const float qs = (sred[(2 * j) * 4] + sred[(2 * j) * 4 + 1]) + (sred[(2 * j) * 4 + 2] + sred[(2 * j) * 4 + 3]);
                    const float ks = (sred[(2 * j + 1) * 4] + sred[(2 * j + 1) * 4 + 1]) + (sred[(2 * j + 1) * 4 + 2] + sred[(2 * j + 1) * 4 + 3]);
                    const float qr = 1.0f / sqrtf(qs / (float)DK + e2);
                    const float kr = 1.0f / sqrtf(ks / (float)DK + e2);
                    sq[j * DK + tid] = bf(bf(qv[j] * qr) * sc_q);          // l2norm(q) / sqrt(128), rounded like kernels.py:504-509
                    sk[j * DK + tid] = bf(bf(kv[j] * kr) * sc_k);
                }
            }
            // (the barrier inside the slice step below orders these writes before their readers)
            if (idx == lo) GDN_BSTAMP(1);
        }

        // ---- state slice: shared memory -> registers, then give the stage back to the copy engine ----
        const bool arrived = sm100::mbar_wait(sm100::smem_addr(&full_bar[stage]), (uint32_t)(n / NST) & 1u);
        if (n < 4) GDN_BSTAMP(2 + 2 * n);
        float4 s[2][4];
        int rows[2];
        const float* sl_base = ring + stage * SLICE_FLOATS;
#pragma unroll
        for (int p = 0; p < 2; p++) {
            rows[p] = (warp * 2 + p) * 4 + sub;                            // row within the slice
#pragma unroll
            for (int i = 0; i < 4; i++) s[p][i] = *reinterpret_cast<const float4*>(sl_base + rows[p] * DK + l8 * 4 + 32 * i);
        }
        __syncthreads();
        if (tid == 0 && idx + NST < hi) {
            // the slice three ahead lies in this head or in the next one, whose pointers are in registers already
            const int ib = (idx + NST) / (HV * SLICES_PER_HEAD);
            issue(idx + NST, ib == cur_b ? sp.st_in : (ib == have_b ? nxt_sp.st_in : resolve(a, ib).st_in));
        }
        if (!arrived) { if (tid == 0) atomicExch(a.status, 2); continue; }
        if (!sp.ok) continue;

        __nv_bfloat16* yb = a.y + (size_t)b * M * (HV * DV) + hv * DV + sl * SLICE_ROWS;
        float* so_head = sp.st_out + ((size_t)hv * DV + sl * SLICE_ROWS) * DK;
        for (int j = 0; j < M; j++) {
            float4 kk[4], qq[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                kk[i] = *reinterpret_cast<const float4*>(sk + j * DK + l8 * 4 + 32 * i);
                qq[i] = *reinterpret_cast<const float4*>(sq + j * DK + l8 * 4 + 32 * i);
            }
            const float g = sgate[2 * j], beta = sgate[2 * j + 1];
            float* so = so_head + (size_t)j * STATE_ELEMS;
#pragma unroll
            for (int p = 0; p < 2; p++) {
                float kvm = 0.f;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    s[p][i].x *= g; s[p][i].y *= g; s[p][i].z *= g; s[p][i].w *= g;
                    kvm += (s[p][i].x * kk[i].x + s[p][i].y * kk[i].y) + (s[p][i].z * kk[i].z + s[p][i].w * kk[i].w);
                }
                kvm += __shfl_xor_sync(0xffffffffu, kvm, 1);
                kvm += __shfl_xor_sync(0xffffffffu, kvm, 2);
                kvm += __shfl_xor_sync(0xffffffffu, kvm, 4);
                const float delta = (sv[j * DV + sl * SLICE_ROWS + rows[p]] - kvm) * beta;
                float yv = 0.f;
                float* rp = so + rows[p] * DK + l8 * 4;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    s[p][i].x += kk[i].x * delta; s[p][i].y += kk[i].y * delta;
                    s[p][i].z += kk[i].z * delta; s[p][i].w += kk[i].w * delta;
                    yv += (s[p][i].x * qq[i].x + s[p][i].y * qq[i].y) + (s[p][i].z * qq[i].z + s[p][i].w * qq[i].w);
                    *reinterpret_cast<float4*>(rp + 32 * i) = s[p][i];
                }
                yv += __shfl_xor_sync(0xffffffffu, yv, 1);
                yv += __shfl_xor_sync(0xffffffffu, yv, 2);
                yv += __shfl_xor_sync(0xffffffffu, yv, 4);
                if (l8 == 0) yb[(size_t)j * (HV * DV) + rows[p]] = __float2bfloat16_rn(yv);
            }
        }
        if (n < 4) GDN_BSTAMP(3 + 2 * n);
        if (idx == hi - 1) GDN_BSTAMP(13);
    }
}

template <int MT>
static int launch_mt(const DecodeArgs& a, cudaStream_t stream) {
    static bool attr_set[64] = {};
    static int sms[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    constexpr int NST = Tune<MT>::NST;
    const int smem = NST * SLICE_BYTES + (3 * MT * DK + 2 * MT * 4 + 2 * MT) * (int)sizeof(float);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        if (cudaFuncSetAttribute(gdn_decode_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return check_launch("gdn_decode smem attribute");
        cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
        attr_set[dev] = true;
    }
    const int n_sm = (dev >= 0 && dev < 64 && sms[dev] > 0) ? sms[dev] : 148;
    const int n_slices = a.B * HV * SLICES_PER_HEAD;
    int grid = Tune<MT>::BLOCKS * n_sm;
    const int n_heads = a.B * HV;
    // small batches: one block per head (4 slices, one prologue, a full ring) beats more blocks with 1-2 slices and a prologue
    // each; very small ones (fewer heads than SMs) fall back to one slice per block so that every SM has work
    if (n_heads <= grid && n_heads >= n_sm) grid = n_heads;
    if (grid > n_slices) grid = n_slices;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid); cfg.blockDim = dim3(128); cfg.dynamicSmemBytes = (size_t)smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    // Early scheduling of the next launch pays when its blocks can only land where blocks of this one leave (every slot taken: they
    // then spread as evenly as these; +2% on the step, with or without host copies beside it) or when every block has an SM to
    // itself (+6-9% at B = 1).  With a partly filled GPU the early blocks pile up on the SMs that happen to have free slots and the
    // launch runs at the pace of its fullest SM (measured: B = 16 15-23% slower), so there it is not asked for.
    attr[0].val.programmaticStreamSerializationAllowed = (grid >= Tune<MT>::BLOCKS * n_sm || grid <= n_sm) ? 1 : 0;
    cfg.attrs = attr; cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, gdn_decode_kernel<MT>, a, n_slices);
    return check_launch("gdn_decode");
}

int launch_decode(const DecodeArgs& a, cudaStream_t stream) {
    if (a.B <= 0 || a.M <= 0) return GDN_OK;
    if (a.M == 1) return launch_mt<1>(a, stream);
    if (a.M <= 4) return launch_mt<4>(a, stream);
    if (a.M <= 8) return launch_mt<8>(a, stream);
    set_error("gdn_decode: M = %d chained tokens exceeds the supported 8", a.M);
    return GDN_E_SHAPE;
}

}  // namespace gdn

#ifdef GDN_TIMING
extern "C" __attribute__((visibility("default"))) int gdn_timing_log_e(long long* out_host, int n) {
    return cudaMemcpyFromSymbol(out_host, gdn::g_tlog, sizeof(long long) * n) == cudaSuccess ? 0 : -5;
}
#endif
