/* libgdn_b200 -- C ABI of the B200 (sm_100a) GatedDeltaNet / GQA-decode kernels.
 *
 * The reference project (a Python/MLX code base) has no FFI layer: its operators are Python functions that JIT-compile
 * Metal source.  Each entry point below is what a binding for one of those operators calls; the comment on each names
 * the reference function it stands in for (paths relative to the reference project root).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless the name ends in `_host`; bf16 tensors are passed as `void*`
 *   - every function only enqueues work on `stream` (a cudaStream_t passed as void*; NULL = default stream); nothing
 *     synchronises, allocates or retains caller memory
 *   - the return value is 0 on success or one of the negative GDN_E_* codes; `gdn_last_error_string()` describes the last
 *     failure of the calling thread.  Index arrays that live on the device (slots, positions, block tables) cannot be
 *     checked by the host: the kernels range-check them, skip the offending row and set a device status word that
 *     `gdn_device_status()` reads back.
 *   - model constants: 16 heads, d_k = d_v = 128, mixed-qkv width 6144, in_proj row 8224 (qkv | z 2048 | b 16 | a 16),
 *     one recurrent state = fp32 [16][128 value rows][128 key columns]
 */
#ifndef GDN_B200_H
#define GDN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* The library is built with hidden visibility; only the entry points declared here are exported. */
#if defined(__GNUC__)
#define GDN_API __attribute__((visibility("default")))
#else
#define GDN_API
#endif

#define GDN_OK 0
#define GDN_E_SHAPE (-1)
#define GDN_E_DTYPE (-2)
#define GDN_E_ALIGN (-3)
#define GDN_E_INDEX (-4)
#define GDN_E_LAUNCH (-5)
#define GDN_E_TIMEOUT (-6)
#define GDN_E_UNSUPPORTED (-7)
#define GDN_E_NULL (-8)

/* Library version (major*10000 + minor*100 + patch). */
GDN_API int gdn_version(void);

/* Message of the last error returned to the calling thread ("" if none). */
GDN_API const char* gdn_last_error_string(void);

/* Reads (and clears) the current device's status word.  Synchronises the device.  Values (the last event wins):
 *   0  every device-side check passed since the last call
 *   1  a slot / snapshot / page index or a cu_seqlens entry was out of range: that row (sequence) was skipped, or, for a page
 *      index inside a context, page 0 was read in its place and that sequence's attention output is undefined
 *   2  a bounded wait inside the decode or attention kernel gave up (its copies never arrived); the block left early
 *   3  a bounded wait inside a prefill kernel gave up; the block left early
 *   4  a kernel found its dynamic shared memory not 1024-byte aligned and did nothing
 * None of these faults the device: the context stays usable and the affected outputs are left unwritten or undefined. */
GDN_API int gdn_device_status(int* status_host);

/* compute_g and beta = sigmoid(b) with the reference's bf16 rounding points.
 * Replaces: compute_g, qwen35/gated_delta.py:16-18; beta at qwen35/gated_delta.py:158; kernel form qwen35/kernels.py:511-515.
 *   a, b     bf16, element (row r, head h) at a[r*a_stride + h] / b[r*b_stride + h]   (either may be NULL)
 *   A_log, dt_bias   fp32 [H]
 *   g, lg, beta      fp32 [n_rows, H] outputs: decay exp(lg), log-decay, beta           (any may be NULL) */
GDN_API int gdn_gates(const void* a, const void* b, long long a_stride, long long b_stride, const float* A_log, const float* dt_bias,
              float* g, float* lg, float* beta, long long n_rows, int H, void* stream);

/* q <- l2norm(q) * inv_scale^2, k <- l2norm(k) * inv_scale over rows of 128 bf16.
 * Replaces: normalize_qk, qwen35/gated_delta.py:21-30 (kernel form qwen35/kernels.py:490-509). */
GDN_API int gdn_normalize_qk(const void* q, const void* k, void* q_out, void* k_out, long long n_rows, float inv_scale, float eps, void* stream);

/* Sequential gated delta rule over T tokens.
 * Replaces: gated_delta_update's kernel, qwen35/gated_delta.py:33-137,167-174.
 *   q, k  bf16 [B,T,Hk,128];  v bf16 [B,T,Hv,Dv];  g, beta fp32 [B,T,Hv];  state_in fp32 [B,Hv,Dv,128] or NULL (zeros)
 *   y     bf16 [B,T,Hv,Dv];   state_out fp32 [B,Hv,Dv,128]
 * Errors: GDN_E_SHAPE unless Dk == 128, Dv % 16 == 0 and Hv % Hk == 0 (the reference raises ValueError, gated_delta.py:164-166). */
GDN_API int gdn_recurrent(const void* q, const void* k, const void* v, const float* g, const float* beta, const float* state_in, void* y,
                  float* state_out, int B, int T, int Hk, int Hv, int Dk, int Dv, void* stream);

/* Chunked prefill (chunk 64, tcgen05 tensor cores) over a packed varlen batch, with optional resume from a cached state:
 * phase A followed by phase B (the two entry points below), as the reference's gdn_chunked is its two kernels back to back.
 * Replaces: gdn_chunked, qwen35/gdn_nax.py:413-426.  The reference handles one sequence per call (B = 1); cu_seqlens packing
 * and init_idx are the additive extension for ragged batches and prefix-cache resume.
 *   q, k, v  bf16 [total_T, H, 128] (q, k already normalised; q scaled by 128^-1/2), 16-byte aligned
 *   lg, beta fp32 [total_T, H]: log-decay and beta of every token and head (see gdn_gates)
 *   cu_seqlens int32 [n_seq+1] (device): sequence s owns tokens [cu_seqlens[s], cu_seqlens[s+1])
 *   init_state fp32 [*, H, 128, 128] or NULL (zero states); init_idx int32 [n_seq] (device) or NULL: row of init_state the
 *              sequence resumes from, negative = zero state; with init_state != NULL and init_idx == NULL row s is used
 *   y bf16 [total_T, H, 128];  final_state fp32 [n_seq, H, 128, 128]
 *   workspace: gdn_prefill_workspace_bytes(n_seq, total_T, H) bytes, 16-byte aligned: the phase-A records between the two kernels
 *   heads [head_lo, head_hi) are computed (head-group sharding of one long sequence); the others are not touched
 * Errors: GDN_E_SHAPE for bad sizes or a short workspace, GDN_E_ALIGN, GDN_E_UNSUPPORTED if the driver lacks tensor-map support. */
GDN_API int gdn_prefill_chunked(const void* q, const void* k, const void* v, const float* lg, const float* beta, const int* cu_seqlens,
                        const float* init_state, const int* init_idx, void* y, float* final_state, void* workspace, size_t workspace_bytes,
                        int n_seq, long long total_T, int H, int head_lo, int head_hi, void* stream);

/* Bytes of the phase-A record buffer for a packed batch: (total_T / 64 + n_seq) * H records of 17,152 bytes (Tb as bf16 hi + lo
 * operand images, and the chunk's cumulative log-decay, gamma and dec vectors).  Stands in for the reference's Tbuf / Abuf / gv
 * outputs of phase A (qwen35/gdn_nax.py:394-401,420-422). */
GDN_API size_t gdn_prefill_workspace_bytes(int n_seq, long long total_T, int H);

/* Phase A: the state-independent part of every 64-token chunk, one independent tile per (chunk, head) -- cumulative decay,
 * K K^T on the tensor cores, the exact inverse (I + L)^-1 and Tb = T diag(beta) -- written as records for phase B.
 * Replaces: the reference's phase-A kernel gdn_nax_a, qwen35/gdn_nax.py:71-143 (launched at :420-422). */
GDN_API int gdn_phase_a(const void* k, const float* lg, const float* beta, const int* cu_seqlens, void* records, size_t records_bytes, int n_seq,
                long long total_T, int H, int head_lo, int head_hi, void* stream);

/* Phase A fused with the prefill front end: reads the in_proj rows once, computes conv (4 taps) + silu, q / k l2norm (q also scaled
 * by 128^-1/2) and the gates, writes q, k, v for phase B and the phase-A records.  Bit-identical to gdn_conv_prep + gdn_gates +
 * gdn_phase_a.  H is 16 (the in_proj row layout fixes it).
 * Replaces: prep_a, qwen35/gdn_nax.py:394-401 (kernel :150-222), the reference's default prefill path (qwen35/prefill.py:251-252).
 *   proj bf16 [total_T, row_stride >= 8224];  conv_state bf16 [n_seq, 3, 6144]: the three raw rows before each sequence
 *   conv_w bf16 [6144*4];  A_log, dt_bias fp32 [16];  q, k, v bf16 [total_T, 16, 128] outputs */
GDN_API int gdn_prep_a(const void* proj, long long row_stride, const void* conv_state, const void* conv_w, const float* A_log, const float* dt_bias,
               const int* cu_seqlens, void* q, void* k, void* v, void* records, size_t records_bytes, int n_seq, long long total_T, int head_lo,
               int head_hi, void* stream);

/* Phase B: the serial chain over the chunks of every (sequence, head), fp32 state resident in tensor memory.
 * Replaces: phase_b, qwen35/gdn_nax.py:404-410 (kernel gdn_nax_b :224-358), called at qwen35/prefill.py:253. */
GDN_API int gdn_phase_b(const void* q, const void* k, const void* v, const void* records, size_t records_bytes, const int* cu_seqlens,
                const float* init_state, const int* init_idx, void* y, float* final_state, int n_seq, long long total_T, int H, int head_lo,
                int head_hi, void* stream);

/* Causal prefill attention, head_dim 256, 8 query heads on 2 KV heads, on the tensor cores: for the S query tokens at positions
 * pos .. pos + S - 1, out[i, h, :] = softmax(q[i, h, :] . K[0 .. pos + i, h / 4, :] / 16) V[0 .. pos + i, h / 4, :] (fp32 scores and
 * accumulation, bf16 in and out).
 * Replaces: the scaled_dot_product_attention call of the prefill, qwen35/model.py:165 (function :148-169), reached from
 * qwen35/prefill.py:468; the reference passes q [1,8,S,256] and K / V [1,2,kv_len,256] with a causal mask.
 *   q, out bf16 [S, 8, 256];  k, v bf16: key t of KV head g at k + t * k_tok_stride + g * k_head_stride (elements), so both the
 *   reference's [2, T, 256] cache (tok stride 256, head stride T_max * 256) and a [T, 2, 256] layout (512, 256) are accepted; K and V
 *   must use the same kind of layout; keys 0 .. pos + S - 1 must exist.  Strides are multiples of 8 elements, pointers 16-byte aligned.
 *   workspace (optional, may be NULL): with gqa_prefill_attn_workspace_bytes(S, pos) bytes (16-byte aligned, contents need no
 *   initialisation, not shared by calls that overlap on the GPU) the query blocks with the most keys are split in two along the keys
 *   and merged in the kernel, which shortens the launch when S is too small to give every SM several blocks; the function returns 0
 *   bytes for shapes that are not split.  Results with and without a workspace agree to rounding (different summation order). */
GDN_API int gqa_prefill_attn(const void* q, const void* k, const void* v, void* out, int S, int pos, long long k_tok_stride, long long k_head_stride,
                     long long v_tok_stride, long long v_head_stride, void* workspace, size_t workspace_bytes, void* stream);
GDN_API size_t gqa_prefill_attn_workspace_bytes(int S, int pos);

/* Phase B with the gated RMSNorm of the layer fused into its y store: y <- bf16(silu(z) * (gate_w * (y * rsqrt(mean(y^2) + 1e-6))))
 * per (token, head) row, computed on the bf16-rounded y exactly as gdn_gated_norm does (same bits as gdn_phase_b followed by
 * gdn_gated_norm), so the y tensor never makes the round trip through memory between the two.
 * Replaces: phase_b followed by gated_norm, qwen35/prefill.py:253-254 (gated_norm :137-157,241-244).
 *   gate_z bf16: the z slice of the projection rows, element (t, h, c) at gate_z[t * gate_stride + h * 128 + c]
 *   (for in_proj rows: proj + 6144, gate_stride = the row stride); 16-byte aligned rows.  gate_w fp32 [128].
 *   gate_z == gate_w == NULL: plain gdn_phase_b. */
GDN_API int gdn_phase_b_gated(const void* q, const void* k, const void* v, const void* records, size_t records_bytes, const int* cu_seqlens,
                      const float* init_state, const int* init_idx, const void* gate_z, long long gate_stride, const float* gate_w, void* y,
                      float* final_state, int n_seq, long long total_T, int H, int head_lo, int head_hi, void* stream);

/* Decode / speculative verify, solo flavour: M chained tokens, functional snapshot outputs.
 * Replaces: deltanet, qwen35/kernels.py:555-567 (kernel :461-552).
 *   proj bf16 [M, row_stride>=8224];  conv_snap bf16 [n_snap,3,6144];  conv_w bf16 [6144*4];  ssm_snap fp32 [n_snap,16,128,128]
 *   sel int32[1] (device): snapshot the call starts from
 *   y bf16 [M,2048];  conv_out bf16 [M,3,6144];  ssm_out fp32 [M,16,128,128]   (snapshot j = state after token j) */
GDN_API int gdn_deltanet(const void* proj, long long row_stride, const void* conv_snap, const void* conv_w, const float* A_log,
                 const float* dt_bias, const float* ssm_snap, const int* sel, int n_snap, void* y, void* conv_out, float* ssm_out,
                 int M, void* stream);

/* Batched decode, one token for each of B slots, pools updated in place.
 * Replaces: deltanet_b, qwen35/batch.py:128-135 (kernel :36-127).
 *   conv_pool bf16 [n_slots*2,3,6144] (reads buffer pos&1 of the slot, writes the other);  ssm_pool fp32 [n_slots,16,128,128]
 *   slots, pos int32 [B] (device);  y bf16 [B,2048] */
GDN_API int gdn_deltanet_b(const void* proj, long long row_stride, void* conv_pool, const void* conv_w, const float* A_log, const float* dt_bias,
                   float* ssm_pool, const int* slots, const int* pos, int n_slots, void* y, int B, void* stream);

/* Batched speculative verify, M chained tokens for each of B sequences over snapshot pools, in place.
 * Replaces: deltanet_bm, qwen35/batch_spec.py:142-150 (kernel :45-141).
 *   conv_pool bf16 [n_entries*2, M, 3, 6144];  ssm_pool fp32 [n_entries, M, 16,128,128]
 *   sslots, sels, pars int32 [B] (device): pool entry, start snapshot, conv buffer read (the other one is written)
 *   proj bf16 [B*M, row_stride];  y bf16 [B*M,2048] */
GDN_API int gdn_deltanet_bm(const void* proj, long long row_stride, void* conv_pool, const void* conv_w, const float* A_log, const float* dt_bias,
                    float* ssm_pool, const int* sslots, const int* sels, const int* pars, int n_entries, void* y, int B, int M,
                    void* stream);

/* Bytes of fp32 workspace gqa_decode_paged needs for B sequences whose contexts are at most max_ctx tokens. */
GDN_API size_t gqa_decode_workspace_bytes(int B, int max_ctx);

/* GQA decode attention (8 query heads, 2 KV heads, head_dim 256) over a paged bf16 KV cache, M <= 4 chained rows per
 * sequence, new K/V rows appended in place.
 * Replaces: attn_b, qwen35/batch.py:230-237 (kernel :141-227); the reference's slot pool [S+1,2,Lmax,256] is the case
 * page_size = Lmax, max_pages = 1, block_table = slots.
 *   q bf16 [B*M,8,256] (normed + roped, unscaled);  k_new, v_new bf16 [B*M,2,256]
 *   k_pages, v_pages bf16 [n_pages,2,page_size,256];  block_table int32 [B,max_pages];  ctx_len int32 [B] (tokens cached)
 *   out bf16 [B*M,8,256];  workspace: at least gqa_decode_workspace_bytes(B, max_ctx) bytes, 16-byte aligned (GDN_E_SHAPE otherwise)
 *   max_ctx: host-side upper bound of ctx_len (informational: the work split is derived from ctx_len on the device) */
GDN_API int gqa_decode_paged(const void* q, const void* k_new, const void* v_new, void* k_pages, void* v_pages, const int* block_table,
                     const int* ctx_len, void* out, void* workspace, size_t workspace_bytes, int B, int M, int page_size,
                     int max_pages, int n_pages, int max_ctx, void* stream);

/* gqa_decode_paged for callers that cannot provide a workspace because they cannot allocate device memory: an operator
 * plugged into a serving runtime that reserved the whole device up front and forbids allocation calls on its request path, or
 * a plain C caller that has no allocator of its own to size a workspace with.  This entry point has no counterpart in the
 * reference; it exists only for such hosts.  Same arguments and results as gqa_decode_paged, minus the workspace: the
 * work plan and the split-KV partials go to a 12 MiB array built into the library (held by every GPU that loads the library until the process
 * exits).  Nothing is allocated or freed, here or in anything it calls.
 *   Limit: at most 256 sequences per call (the array holds the work plan and 762 partials: one per SM plus one per
 *          (sequence, kv head) pair).  Larger batches return GDN_E_SHAPE with a message that names the limit; use
 *          gqa_decode_paged for them.
 *   First call on a device: looks up the array's device address (cudaGetSymbolAddress, with that device current).  Make that
 *          first call outside any stream capture.
 *   Sharing: all calls on a device use the same array, which keeps the previous call's contents.  Nothing in it needs
 *          clearing between calls, but two calls that run concurrently on one GPU (different streams) corrupt each other. */
GDN_API int gqa_decode_paged_static(const void* q, const void* k_new, const void* v_new, void* k_pages, void* v_pages, const int* block_table,
                            const int* ctx_len, void* out, int B, int M, int page_size, int max_pages, int n_pages, int max_ctx,
                            void* stream);

/* Glue between the qkv projection of a full-attention layer and gqa_decode_paged: per row, split q | gate per head, k, v;
 * rms_norm(q, q_norm) and rms_norm(k, k_norm) over 256; RoPE on dims [0, 64) (pairs i, i+32; angle pos * theta^(-i/32)).
 * Replaces: the MLX calls at qwen35/fast.py:70-78 (= qwen35/batch.py:504-511, qwen35/model.py:148-161).
 *   qkv bf16 [R, row_stride >= 5120] (8 x (q 256 | gate 256), k 2 x 256, v 2 x 256);  q_norm, k_norm fp32 [256] (the "+1" of
 *   the checkpoint already folded in, qwen35/model.py:95-96);  row_pos int32 [R] position of every row
 *   q bf16 [R,8,256], gate bf16 [R,8,256], k, v bf16 [R,2,256] */
GDN_API int gqa_qkv_prep(const void* qkv, long long row_stride, const float* q_norm, const float* k_norm, const int* row_pos, void* q, void* gate, void* k,
                 void* v, int R, float eps, float rope_theta, void* stream);

/* out = o * sigmoid(gate), elementwise over n bf16 values (n % 4 == 0).  Replaces: qwen35/fast.py:84, qwen35/batch.py:512. */
GDN_API int gqa_gate_out(const void* o, const void* gate, void* out, long long n, void* stream);

/* Prefill front end of a GDN layer: depthwise causal conv (4 taps) + silu on the mixed qkv columns of proj, q/k l2norm (q also
 * scaled by 128^-1/2), and the new conv window (last 3 raw rows).
 * Replaces: conv_prep, qwen35/prefill.py:96-134,160-238; window update qwen35/prefill.py:262-263.
 *   proj bf16 [S, row_stride >= 8224];  conv_state bf16 [3,6144];  conv_w bf16 [6144*4]
 *   q, k, v bf16 [S,16,128];  new_conv bf16 [3,6144] (must not alias conv_state) */
GDN_API int gdn_conv_prep(const void* proj, long long row_stride, const void* conv_state, const void* conv_w, void* q, void* k, void* v, void* new_conv,
                  int S, void* stream);

/* Gated RMSNorm on the GDN output: out = silu(z) * w * y * rsqrt(mean(y^2) + 1e-6) per (token, head), z = proj[:, 6144:8192].
 * Replaces: gated_norm, qwen35/prefill.py:137-157,241-244.
 *   y bf16 [S,2048];  proj bf16 [S, row_stride >= 8224];  gw fp32 [128];  out bf16 [S,2048] */
GDN_API int gdn_gated_norm(const void* y, const void* proj, long long row_stride, const float* gw, void* out, long long S, void* stream);

/* dst.flat[d0 + y*dstride + i] = src.flat[s0 + y*sstride + i] for i < n, y < ny; offsets in elements of elem_size (2 or 4) bytes.
 * Replaces: blit, qwen35/batch.py:349-372. */
GDN_API int gdn_state_copy(void* dst, const void* src, int elem_size, long long n, long long d0, long long s0, int ny, long long dstride,
                   long long sstride, void* stream);

/* hist[slots[b], pos[b], :] = rows[b, :] for b < B: the hidden-state history of the speculative mode, written in place.
 * Replaces: hrec, qwen35/batch.py:375-399.
 *   hist bf16 [n_slots, Lh, H];  rows bf16 [B, H];  slots, pos int32 [B] on the device (an out-of-range entry skips its row and sets
 *   device status 1). */
GDN_API int gdn_hrec(void* hist, const void* rows, const int* slots, const int* pos, int B, int n_slots, int Lh, int H, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* GDN_B200_H */
