// Argument blocks and host launchers of the kernels (one translation unit per kernel family).
#pragma once
#include "gdn_common.cuh"

namespace gdn {

// ---- gdn_decode.cu ----
struct DecodeArgs {
    const __nv_bfloat16* proj;        // [B*M, row_stride] rows: qkv 6144 | z 2048 | b 16 | a 16
    long long row_stride;             // elements between consecutive proj rows
    __nv_bfloat16* conv_pool;         // conv windows (layout depends on mode)
    const __nv_bfloat16* conv_w;      // [6144*4] flat ch*4+tap, tap 3 = current token
    const float* A_log;               // [16]
    const float* dt_bias;             // [16]
    float* ssm_pool;                  // fp32 states (layout depends on mode)
    const int* i0;                    // mode 0: sel[1]      mode 1: slots[B]   mode 2: sslots[B]
    const int* i1;                    //                     mode 1: pos[B]     mode 2: sels[B]
    const int* i2;                    //                                        mode 2: pars[B]
    __nv_bfloat16* y;                 // [B*M, 2048]
    __nv_bfloat16* conv_out;          // mode 0: [M,3,6144]
    float* ssm_out;                   // mode 0: [M,16,128,128]
    int* status;                      // device word: set to 1 if an index was out of range (that row is skipped)
    int B, M, mode, n_entries;        // n_entries: number of snapshots (mode 0) / slots (mode 1) / snapshot-pool entries (mode 2)
};

int launch_decode(const DecodeArgs& a, cudaStream_t stream);

// ---- gdn_recurrent.cu ----
struct RecurrentArgs {
    const __nv_bfloat16 *q, *k, *v;   // q,k [B,T,Hk,128]; v [B,T,Hv,Dv]
    const float *g, *beta;            // [B,T,Hv]
    const float* state_in;            // [B,Hv,Dv,128] or nullptr (zeros)
    __nv_bfloat16* y;                 // [B,T,Hv,Dv]
    float* state_out;                 // [B,Hv,Dv,128]
    int B, T, Hk, Hv, Dv;
};

int launch_recurrent(const RecurrentArgs& a, cudaStream_t stream);
int launch_gates(const __nv_bfloat16* a, const __nv_bfloat16* b, long long a_stride, long long b_stride, const float* A_log,
                 const float* dt_bias, float* g, float* lg, float* beta, long long n_rows, int H, cudaStream_t stream);
int launch_normalize_qk(const __nv_bfloat16* q, const __nv_bfloat16* k, __nv_bfloat16* qo, __nv_bfloat16* ko, long long n_rows,
                        float inv_scale, float eps, cudaStream_t stream);

// ---- gqa_decode.cu ----
struct AttnArgs {
    const __nv_bfloat16 *q, *k_new, *v_new;     // q [B*M,8,256]; k_new, v_new [B*M,2,256]
    __nv_bfloat16 *k_pages, *v_pages;           // [n_pages, 2, page_size, 256]
    const int* block_table;                     // [B, max_pages]
    const int* ctx_len;                         // [B] tokens already cached
    __nv_bfloat16* out;                         // [B*M,8,256]
    int* meta;                                  // work plan in the workspace (tile and partial-slot prefix sums per pair)
    float* part;                                // fp32 partials in the workspace: [slots][PART_STRIDE]
    int* status;
    int B, M, page_size, max_pages, n_pages;
    int P, G;                                   // pairs (= 2 B) and persistent blocks; filled in by the launcher
    int tail_tiles;                             // plan weight of a pair's epilogue, in tiles (filled in by the launcher)
};

size_t gqa_workspace_bytes(int B, int max_ctx);
int launch_gqa_decode(AttnArgs a, void* workspace, size_t workspace_bytes, cudaStream_t stream);
int launch_gqa_decode_static(AttnArgs a, cudaStream_t stream);

// ---- gdn_phase_a.cu / gdn_prefill_sm100.cu ----
constexpr int PA_REC_BYTES = 17152;   // one phase-A record: Tb hi + Tb lo (2 x 8 KiB operand images) + Lc, gamma, dec ([64] fp32 each)

struct PhaseAArgs {
    const float* lg;                  // [total_T, H] log-decay per token and head            (plain flavour)
    const float* beta;                // [total_T, H]
    const int* cu_seqlens;            // [n_seq + 1]
    unsigned char* records;           // [total_T / 64 + n_seq][H] records of PA_REC_BYTES
    int* status;
    int n_seq, H, head_lo, n_heads;
    long long total_T;
    // fused flavour: q, k, v, the gates and the records all come from the in_proj rows
    const __nv_bfloat16* proj;        // [total_T, row_stride] rows: qkv 6144 | z 2048 | b 16 | a 16
    long long row_stride;
    const __nv_bfloat16* conv_state;  // [n_seq, 3, 6144] raw rows before each sequence
    const __nv_bfloat16* conv_w;      // [6144*4]
    const float* A_log;               // [16]
    const float* dt_bias;             // [16]
    __nv_bfloat16 *q, *k, *v;         // [total_T, 16, 128] outputs
};
long long phase_a_slots(int n_seq, long long total_T);
size_t prefill_records_bytes(int n_seq, long long total_T, int H);
int launch_phase_a(const void* k, const PhaseAArgs& a, bool fused, cudaStream_t stream);

struct PrefillArgs {
    const unsigned char* records;     // phase-A records (see PhaseAArgs)
    const int* cu_seqlens;            // [n_seq + 1] token offsets of the packed sequences
    const float* init_state;          // [*, H, 128, 128] fp32 or nullptr (all sequences start from zero)
    const int* init_idx;              // [n_seq] row of init_state per sequence (< 0 = zero state) or nullptr (row = sequence)
    __nv_bfloat16* y;                 // [total_T, H, 128]
    float* final_state;               // [n_seq, H, 128, 128]
    int* status;
    int n_seq, H, head_lo, n_heads;
    long long total_T;
    // optional gated RMSNorm fused into the y store (gate_w != nullptr): y <- silu(z) * rmsnorm(y) * gate_w with
    // z = gate_z[t * gate_stride + h * 128 + c] (the z slice of the projection row of token t)
    const __nv_bfloat16* gate_z;
    long long gate_stride;
    const float* gate_w;              // [128] fp32
};
int launch_phase_b(const void* q, const void* k, const void* v, const PrefillArgs& a, cudaStream_t stream);

// ---- attn_glue.cu ----
int launch_qkv_prep(const __nv_bfloat16* qkv, long long row_stride, const float* q_norm, const float* k_norm, const int* row_pos, __nv_bfloat16* q,
                    __nv_bfloat16* gate, __nv_bfloat16* k, __nv_bfloat16* v, int R, float eps, float theta, cudaStream_t st);
int launch_gate_out(const __nv_bfloat16* o, const __nv_bfloat16* gate, __nv_bfloat16* out, long long n, cudaStream_t st);
int launch_conv_prep(const __nv_bfloat16* proj, long long row_stride, const __nv_bfloat16* conv_state, const __nv_bfloat16* conv_w, __nv_bfloat16* q,
                     __nv_bfloat16* k, __nv_bfloat16* v, __nv_bfloat16* new_conv, int S, cudaStream_t st);
int launch_gated_norm(const __nv_bfloat16* y, const __nv_bfloat16* proj, long long row_stride, const float* gw, __nv_bfloat16* out, long long S,
                      cudaStream_t st);

// ---- gqa_prefill_tc.cu ----
int launch_gqa_prefill(const void* q, const void* k, const void* v, void* out, int S, int pos, long long k_tok_stride, long long k_head_stride,
                       long long v_tok_stride, long long v_head_stride, void* workspace, size_t workspace_bytes, int* status, cudaStream_t stream);
size_t gqa_prefill_workspace_bytes(int S, int pos);

// ---- state_copy.cu ----
int launch_hrec(void* hist, const void* rows, const int* slots, const int* pos, int B, int n_slots, int Lh, int H, int* status, cudaStream_t st);
int launch_state_copy(void* dst, const void* src, int elem_size, long long n, long long d0, long long s0, int ny, long long dstride,
                      long long sstride, cudaStream_t st);

}  // namespace gdn
