// extern "C" surface of libgdn_b200: argument validation, error strings, and dispatch to the kernel launchers.
#include "../../include/gdn_b200.h"
#include "gdn_common.cuh"
#include "launchers.cuh"

#include <cstdarg>
#include <cstdio>

namespace gdn {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int check_launch(const char* what) {
    const cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return GDN_OK;
    set_error("%s: %s", what, cudaGetErrorString(e));
    return GDN_E_LAUNCH;
}

// one status word per device, written by kernels that skip a row with a bad index
__device__ int g_status_word;


static int* status_ptr() {
    static int* ptrs[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!ptrs[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        ptrs[dev] = static_cast<int*>(p);
    }
    return ptrs[dev];
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace gdn

using namespace gdn;

#define REQUIRE(cond, code, ...) \
    do { if (!(cond)) { set_error(__VA_ARGS__); return (code); } } while (0)

extern "C" {

int gdn_version(void) { return 100; }

const char* gdn_last_error_string(void) { return g_err; }

int gdn_device_status(int* status_host) {
    REQUIRE(status_host, GDN_E_NULL, "gdn_device_status: null output");
    int* p = status_ptr();
    REQUIRE(p, GDN_E_LAUNCH, "gdn_device_status: no CUDA device");
    int zero = 0;
    if (cudaMemcpy(status_host, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess ||
        cudaMemcpy(p, &zero, sizeof(int), cudaMemcpyHostToDevice) != cudaSuccess)
        return check_launch("gdn_device_status");
    return GDN_OK;
}

int gdn_gates(const void* a, const void* b, long long a_stride, long long b_stride, const float* A_log, const float* dt_bias, float* g,
              float* lg, float* beta, long long n_rows, int H, void* stream) {
    REQUIRE(n_rows >= 0 && H > 0, GDN_E_SHAPE, "gdn_gates: n_rows=%lld H=%d", n_rows, H);
    REQUIRE(!a || (A_log && dt_bias), GDN_E_NULL, "gdn_gates: A_log / dt_bias missing");
    return launch_gates(static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), a_stride, b_stride, A_log, dt_bias,
                        g, lg, beta, n_rows, H, static_cast<cudaStream_t>(stream));
}

int gdn_normalize_qk(const void* q, const void* k, void* q_out, void* k_out, long long n_rows, float inv_scale, float eps, void* stream) {
    REQUIRE(q && k && q_out && k_out, GDN_E_NULL, "gdn_normalize_qk: null pointer");
    REQUIRE(n_rows >= 0, GDN_E_SHAPE, "gdn_normalize_qk: n_rows=%lld", n_rows);
    REQUIRE(((uintptr_t)q | (uintptr_t)k | (uintptr_t)q_out | (uintptr_t)k_out) % 8 == 0, GDN_E_ALIGN, "gdn_normalize_qk: rows must be 8-byte aligned");
    return launch_normalize_qk(static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), static_cast<__nv_bfloat16*>(q_out),
                               static_cast<__nv_bfloat16*>(k_out), n_rows, inv_scale, eps, static_cast<cudaStream_t>(stream));
}

int gdn_recurrent(const void* q, const void* k, const void* v, const float* g, const float* beta, const float* state_in, void* y,
                  float* state_out, int B, int T, int Hk, int Hv, int Dk, int Dv, void* stream) {
    REQUIRE(Dk == 128 && Dv > 0 && Dv % 16 == 0 && Hk > 0 && Hv > 0 && Hv % Hk == 0, GDN_E_SHAPE,
            "gdn_recurrent: only Dk=128, Dv%%16==0, Hv%%Hk==0 is supported (Dk=%d, Dv=%d, Hk=%d, Hv=%d)", Dk, Dv, Hk, Hv);
    REQUIRE(B >= 0 && T >= 0, GDN_E_SHAPE, "gdn_recurrent: B=%d T=%d", B, T);
    REQUIRE(q && k && v && g && beta && y && state_out, GDN_E_NULL, "gdn_recurrent: null pointer");
    REQUIRE(aligned16(state_in) && aligned16(state_out) && ((uintptr_t)q | (uintptr_t)k) % 8 == 0, GDN_E_ALIGN, "gdn_recurrent: misaligned tensor");
    RecurrentArgs a{static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), g, beta,
                    state_in, static_cast<__nv_bfloat16*>(y), state_out, B, T, Hk, Hv, Dv};
    return launch_recurrent(a, static_cast<cudaStream_t>(stream));
}

size_t gdn_prefill_workspace_bytes(int n_seq, long long total_T, int H) {
    if (n_seq <= 0 || total_T < 0 || H <= 0) return 0;
    return prefill_records_bytes(n_seq, total_T, H);
}

static int prefill_common(const char* who, const int* cu_seqlens, const void* records, size_t records_bytes, int n_seq, long long total_T, int H,
                          int head_lo, int head_hi) {
    REQUIRE(cu_seqlens && records, GDN_E_NULL, "%s: null pointer", who);
    REQUIRE(n_seq >= 0 && total_T >= 0 && total_T < (1ll << 31) && H > 0 && H <= 65535, GDN_E_SHAPE, "%s: n_seq=%d total_T=%lld H=%d", who, n_seq,
            total_T, H);
    REQUIRE(head_lo >= 0 && head_lo <= head_hi && head_hi <= H, GDN_E_SHAPE, "%s: head range [%d, %d) outside [0, %d)", who, head_lo, head_hi, H);
    REQUIRE(aligned16(records), GDN_E_ALIGN, "%s: the record buffer must be 16-byte aligned", who);
    REQUIRE(records_bytes >= prefill_records_bytes(n_seq, total_T, H), GDN_E_SHAPE, "%s: record buffer of %zu bytes < %zu (gdn_prefill_workspace_bytes)",
            who, records_bytes, prefill_records_bytes(n_seq, total_T, H));
    return GDN_OK;
}

int gdn_phase_a(const void* k, const float* lg, const float* beta, const int* cu_seqlens, void* records, size_t records_bytes, int n_seq,
                long long total_T, int H, int head_lo, int head_hi, void* stream) {
    REQUIRE(k && lg && beta, GDN_E_NULL, "gdn_phase_a: null pointer");
    int rc = prefill_common("gdn_phase_a", cu_seqlens, records, records_bytes, n_seq, total_T, H, head_lo, head_hi);
    if (rc) return rc;
    REQUIRE(aligned16(k), GDN_E_ALIGN, "gdn_phase_a: k must be 16-byte aligned");
    if (n_seq == 0 || head_lo == head_hi || total_T == 0) return GDN_OK;
    PhaseAArgs a{};
    a.lg = lg; a.beta = beta; a.cu_seqlens = cu_seqlens; a.records = static_cast<unsigned char*>(records);
    a.n_seq = n_seq; a.H = H; a.head_lo = head_lo; a.n_heads = head_hi - head_lo; a.total_T = total_T;
    a.status = status_ptr();
    REQUIRE(a.status, GDN_E_LAUNCH, "gdn_phase_a: no CUDA device");
    return launch_phase_a(k, a, false, static_cast<cudaStream_t>(stream));
}

int gdn_prep_a(const void* proj, long long row_stride, const void* conv_state, const void* conv_w, const float* A_log, const float* dt_bias,
               const int* cu_seqlens, void* q, void* k, void* v, void* records, size_t records_bytes, int n_seq, long long total_T, int head_lo,
               int head_hi, void* stream) {
    REQUIRE(proj && conv_state && conv_w && A_log && dt_bias && q && k && v, GDN_E_NULL, "gdn_prep_a: null pointer");
    int rc = prefill_common("gdn_prep_a", cu_seqlens, records, records_bytes, n_seq, total_T, HV, head_lo, head_hi);
    if (rc) return rc;
    REQUIRE(row_stride >= PW && row_stride % 4 == 0, GDN_E_SHAPE, "gdn_prep_a: proj row stride %lld (need >= 8224 and a multiple of 4)", row_stride);
    REQUIRE(((uintptr_t)proj | (uintptr_t)conv_state | (uintptr_t)conv_w | (uintptr_t)q | (uintptr_t)k | (uintptr_t)v) % 8 == 0, GDN_E_ALIGN,
            "gdn_prep_a: tensors must be 8-byte aligned");
    if (n_seq == 0 || head_lo == head_hi || total_T == 0) return GDN_OK;
    PhaseAArgs a{};
    a.cu_seqlens = cu_seqlens; a.records = static_cast<unsigned char*>(records);
    a.n_seq = n_seq; a.H = HV; a.head_lo = head_lo; a.n_heads = head_hi - head_lo; a.total_T = total_T;
    a.proj = static_cast<const __nv_bfloat16*>(proj); a.row_stride = row_stride;
    a.conv_state = static_cast<const __nv_bfloat16*>(conv_state); a.conv_w = static_cast<const __nv_bfloat16*>(conv_w);
    a.A_log = A_log; a.dt_bias = dt_bias;
    a.q = static_cast<__nv_bfloat16*>(q); a.k = static_cast<__nv_bfloat16*>(k); a.v = static_cast<__nv_bfloat16*>(v);
    a.status = status_ptr();
    REQUIRE(a.status, GDN_E_LAUNCH, "gdn_prep_a: no CUDA device");
    return launch_phase_a(nullptr, a, true, static_cast<cudaStream_t>(stream));
}

int gdn_phase_b(const void* q, const void* k, const void* v, const void* records, size_t records_bytes, const int* cu_seqlens,
                const float* init_state, const int* init_idx, void* y, float* final_state, int n_seq, long long total_T, int H, int head_lo,
                int head_hi, void* stream) {
    return gdn_phase_b_gated(q, k, v, records, records_bytes, cu_seqlens, init_state, init_idx, nullptr, 0, nullptr, y, final_state, n_seq, total_T, H,
                             head_lo, head_hi, stream);
}

int gdn_phase_b_gated(const void* q, const void* k, const void* v, const void* records, size_t records_bytes, const int* cu_seqlens,
                      const float* init_state, const int* init_idx, const void* gate_z, long long gate_stride, const float* gate_w, void* y,
                      float* final_state, int n_seq, long long total_T, int H, int head_lo, int head_hi, void* stream) {
    REQUIRE(q && k && v && y && final_state, GDN_E_NULL, "gdn_phase_b: null pointer");
    REQUIRE((gate_z == nullptr) == (gate_w == nullptr), GDN_E_NULL, "gdn_phase_b_gated: gate_z and gate_w go together");
    REQUIRE(!gate_w || (gate_stride >= (long long)H * 128 && gate_stride % 8 == 0 && aligned16(gate_z) && aligned16(gate_w)), GDN_E_ALIGN,
            "gdn_phase_b_gated: gate rows must be 16-byte aligned (stride %lld elements)", gate_stride);
    int rc = prefill_common("gdn_phase_b", cu_seqlens, records, records_bytes, n_seq, total_T, H, head_lo, head_hi);
    if (rc) return rc;
    REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(init_state) && aligned16(final_state), GDN_E_ALIGN,
            "gdn_phase_b: q / k / v / states must be 16-byte aligned");
    if (n_seq == 0 || head_lo == head_hi) return GDN_OK;
    PrefillArgs a{};
    a.records = static_cast<const unsigned char*>(records);
    a.cu_seqlens = cu_seqlens; a.init_state = init_state; a.init_idx = init_idx;
    a.y = static_cast<__nv_bfloat16*>(y); a.final_state = final_state;
    a.n_seq = n_seq; a.H = H; a.head_lo = head_lo; a.n_heads = head_hi - head_lo;
    a.gate_z = static_cast<const __nv_bfloat16*>(gate_z); a.gate_stride = gate_stride; a.gate_w = gate_w;
    a.status = status_ptr();
    REQUIRE(a.status, GDN_E_LAUNCH, "gdn_phase_b: no CUDA device");
    a.total_T = total_T == 0 ? 1 : total_T;     // a tensor map needs a non-empty extent; empty sequences never issue a copy
    return launch_phase_b(q, k, v, a, static_cast<cudaStream_t>(stream));
}

int gdn_prefill_chunked(const void* q, const void* k, const void* v, const float* lg, const float* beta, const int* cu_seqlens,
                        const float* init_state, const int* init_idx, void* y, float* final_state, void* workspace, size_t workspace_bytes,
                        int n_seq, long long total_T, int H, int head_lo, int head_hi, void* stream) {
    int rc = gdn_phase_a(k, lg, beta, cu_seqlens, workspace, workspace_bytes, n_seq, total_T, H, head_lo, head_hi, stream);
    if (rc) return rc;
    return gdn_phase_b(q, k, v, workspace, workspace_bytes, cu_seqlens, init_state, init_idx, y, final_state, n_seq, total_T, H, head_lo, head_hi,
                       stream);
}

static int decode_common(DecodeArgs& a, void* stream, const char* who) {
    REQUIRE(a.proj && a.conv_pool && a.conv_w && a.A_log && a.dt_bias && a.ssm_pool && a.i0 && a.y, GDN_E_NULL, "%s: null pointer", who);
    REQUIRE(a.row_stride >= PW, GDN_E_SHAPE, "%s: proj row stride %lld < 8224", who, a.row_stride);
    REQUIRE(a.B >= 0 && a.M >= 0 && a.M <= 16, GDN_E_SHAPE, "%s: B=%d M=%d (M <= 16)", who, a.B, a.M);
    REQUIRE(a.n_entries > 0, GDN_E_SHAPE, "%s: empty pool", who);
    REQUIRE(aligned16(a.ssm_pool) && aligned16(a.ssm_out) && ((uintptr_t)a.conv_w % 8 == 0), GDN_E_ALIGN, "%s: state must be 16-byte aligned", who);
    a.status = status_ptr();
    REQUIRE(a.status, GDN_E_LAUNCH, "%s: no CUDA device", who);
    return launch_decode(a, static_cast<cudaStream_t>(stream));
}

int gdn_deltanet(const void* proj, long long row_stride, const void* conv_snap, const void* conv_w, const float* A_log, const float* dt_bias,
                 const float* ssm_snap, const int* sel, int n_snap, void* y, void* conv_out, float* ssm_out, int M, void* stream) {
    REQUIRE(conv_out && ssm_out, GDN_E_NULL, "gdn_deltanet: null output");
    DecodeArgs a{};
    a.proj = static_cast<const __nv_bfloat16*>(proj); a.row_stride = row_stride;
    a.conv_pool = const_cast<__nv_bfloat16*>(static_cast<const __nv_bfloat16*>(conv_snap));
    a.conv_w = static_cast<const __nv_bfloat16*>(conv_w); a.A_log = A_log; a.dt_bias = dt_bias;
    a.ssm_pool = const_cast<float*>(ssm_snap); a.i0 = sel;
    a.y = static_cast<__nv_bfloat16*>(y); a.conv_out = static_cast<__nv_bfloat16*>(conv_out); a.ssm_out = ssm_out;
    a.B = 1; a.M = M; a.mode = 0; a.n_entries = n_snap;
    return decode_common(a, stream, "gdn_deltanet");
}

int gdn_deltanet_b(const void* proj, long long row_stride, void* conv_pool, const void* conv_w, const float* A_log, const float* dt_bias,
                   float* ssm_pool, const int* slots, const int* pos, int n_slots, void* y, int B, void* stream) {
    REQUIRE(pos, GDN_E_NULL, "gdn_deltanet_b: null pos");
    DecodeArgs a{};
    a.proj = static_cast<const __nv_bfloat16*>(proj); a.row_stride = row_stride;
    a.conv_pool = static_cast<__nv_bfloat16*>(conv_pool); a.conv_w = static_cast<const __nv_bfloat16*>(conv_w);
    a.A_log = A_log; a.dt_bias = dt_bias; a.ssm_pool = ssm_pool; a.i0 = slots; a.i1 = pos;
    a.y = static_cast<__nv_bfloat16*>(y);
    a.B = B; a.M = 1; a.mode = 1; a.n_entries = n_slots;
    return decode_common(a, stream, "gdn_deltanet_b");
}

int gdn_deltanet_bm(const void* proj, long long row_stride, void* conv_pool, const void* conv_w, const float* A_log, const float* dt_bias,
                    float* ssm_pool, const int* sslots, const int* sels, const int* pars, int n_entries, void* y, int B, int M, void* stream) {
    REQUIRE(sels && pars, GDN_E_NULL, "gdn_deltanet_bm: null sels / pars");
    REQUIRE(M >= 1, GDN_E_SHAPE, "gdn_deltanet_bm: M=%d", M);
    DecodeArgs a{};
    a.proj = static_cast<const __nv_bfloat16*>(proj); a.row_stride = row_stride;
    a.conv_pool = static_cast<__nv_bfloat16*>(conv_pool); a.conv_w = static_cast<const __nv_bfloat16*>(conv_w);
    a.A_log = A_log; a.dt_bias = dt_bias; a.ssm_pool = ssm_pool; a.i0 = sslots; a.i1 = sels; a.i2 = pars;
    a.y = static_cast<__nv_bfloat16*>(y);
    a.B = B; a.M = M; a.mode = 2; a.n_entries = n_entries;
    return decode_common(a, stream, "gdn_deltanet_bm");
}

size_t gqa_decode_workspace_bytes(int B, int max_ctx) {
    if (B <= 0 || max_ctx < 0) return 0;
    return gqa_workspace_bytes(B, max_ctx);
}

int gqa_decode_paged(const void* q, const void* k_new, const void* v_new, void* k_pages, void* v_pages, const int* block_table,
                     const int* ctx_len, void* out, void* workspace, size_t workspace_bytes, int B, int M, int page_size, int max_pages,
                     int n_pages, int max_ctx, void* stream) {
    REQUIRE(q && k_new && v_new && k_pages && v_pages && block_table && ctx_len && out && workspace, GDN_E_NULL, "gqa_decode_paged: null pointer");
    REQUIRE(B >= 0 && M >= 1 && M <= 4, GDN_E_SHAPE, "gqa_decode_paged: B=%d M=%d (1 <= M <= 4)", B, M);
    REQUIRE(page_size > 0 && max_pages > 0 && n_pages > 0 && max_ctx >= 0, GDN_E_SHAPE, "gqa_decode_paged: page_size=%d max_pages=%d n_pages=%d max_ctx=%d",
            page_size, max_pages, n_pages, max_ctx);
    REQUIRE(aligned16(q) && aligned16(k_new) && aligned16(v_new) && aligned16(k_pages) && aligned16(v_pages) && aligned16(out) && aligned16(workspace),
            GDN_E_ALIGN, "gqa_decode_paged: tensors must be 16-byte aligned");
    REQUIRE(workspace_bytes >= gqa_workspace_bytes(B, max_ctx), GDN_E_SHAPE, "gqa_decode_paged: workspace %zu < %zu bytes", workspace_bytes,
            gqa_workspace_bytes(B, max_ctx));
    AttnArgs a{};
    a.q = static_cast<const __nv_bfloat16*>(q); a.k_new = static_cast<const __nv_bfloat16*>(k_new); a.v_new = static_cast<const __nv_bfloat16*>(v_new);
    a.k_pages = static_cast<__nv_bfloat16*>(k_pages); a.v_pages = static_cast<__nv_bfloat16*>(v_pages);
    a.block_table = block_table; a.ctx_len = ctx_len; a.out = static_cast<__nv_bfloat16*>(out);
    a.B = B; a.M = M; a.page_size = page_size; a.max_pages = max_pages; a.n_pages = n_pages;
    a.status = status_ptr();
    REQUIRE(a.status, GDN_E_LAUNCH, "gqa_decode_paged: no CUDA device");
    return launch_gqa_decode(a, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

int gqa_decode_paged_static(const void* q, const void* k_new, const void* v_new, void* k_pages, void* v_pages, const int* block_table,
                            const int* ctx_len, void* out, int B, int M, int page_size, int max_pages, int n_pages, int max_ctx, void* stream) {
    REQUIRE(q && k_new && v_new && k_pages && v_pages && block_table && ctx_len && out, GDN_E_NULL, "gqa_decode_paged_static: null pointer");
    REQUIRE(B >= 0 && M >= 1 && M <= 4, GDN_E_SHAPE, "gqa_decode_paged_static: B=%d M=%d (1 <= M <= 4)", B, M);
    REQUIRE(page_size > 0 && max_pages > 0 && n_pages > 0 && max_ctx >= 0, GDN_E_SHAPE,
            "gqa_decode_paged_static: page_size=%d max_pages=%d n_pages=%d max_ctx=%d", page_size, max_pages, n_pages, max_ctx);
    REQUIRE(aligned16(q) && aligned16(k_new) && aligned16(v_new) && aligned16(k_pages) && aligned16(v_pages) && aligned16(out), GDN_E_ALIGN,
            "gqa_decode_paged_static: tensors must be 16-byte aligned");
    AttnArgs a{};
    a.q = static_cast<const __nv_bfloat16*>(q); a.k_new = static_cast<const __nv_bfloat16*>(k_new); a.v_new = static_cast<const __nv_bfloat16*>(v_new);
    a.k_pages = static_cast<__nv_bfloat16*>(k_pages); a.v_pages = static_cast<__nv_bfloat16*>(v_pages);
    a.block_table = block_table; a.ctx_len = ctx_len; a.out = static_cast<__nv_bfloat16*>(out);
    a.B = B; a.M = M; a.page_size = page_size; a.max_pages = max_pages; a.n_pages = n_pages;
    a.status = status_ptr();
    REQUIRE(a.status, GDN_E_LAUNCH, "gqa_decode_paged_static: no CUDA device");
    return launch_gqa_decode_static(a, static_cast<cudaStream_t>(stream));
}

int gqa_qkv_prep(const void* qkv, long long row_stride, const float* q_norm, const float* k_norm, const int* row_pos, void* q, void* gate, void* k,
                 void* v, int R, float eps, float rope_theta, void* stream) {
    REQUIRE(qkv && q_norm && k_norm && row_pos && q && gate && k && v, GDN_E_NULL, "gqa_qkv_prep: null pointer");
    REQUIRE(R >= 0 && row_stride >= 5120 && rope_theta > 1.f, GDN_E_SHAPE, "gqa_qkv_prep: R=%d row_stride=%lld theta=%g", R, row_stride, rope_theta);
    typedef const __nv_bfloat16* cb; typedef __nv_bfloat16* b;
    return launch_qkv_prep((cb)qkv, row_stride, q_norm, k_norm, row_pos, (b)q, (b)gate, (b)k, (b)v, R, eps, rope_theta, static_cast<cudaStream_t>(stream));
}

int gqa_gate_out(const void* o, const void* gate, void* out, long long n, void* stream) {
    REQUIRE(o && gate && out, GDN_E_NULL, "gqa_gate_out: null pointer");
    REQUIRE(n >= 0 && n % 4 == 0, GDN_E_SHAPE, "gqa_gate_out: n=%lld must be a multiple of 4", n);
    REQUIRE(((uintptr_t)o | (uintptr_t)gate | (uintptr_t)out) % 8 == 0, GDN_E_ALIGN, "gqa_gate_out: tensors must be 8-byte aligned");
    return launch_gate_out((const __nv_bfloat16*)o, (const __nv_bfloat16*)gate, (__nv_bfloat16*)out, n, static_cast<cudaStream_t>(stream));
}

size_t gqa_prefill_attn_workspace_bytes(int S, int pos) { return S > 0 && pos >= 0 ? gdn::gqa_prefill_workspace_bytes(S, pos) : 0; }

int gqa_prefill_attn(const void* q, const void* k, const void* v, void* out, int S, int pos, long long k_tok_stride, long long k_head_stride,
                     long long v_tok_stride, long long v_head_stride, void* workspace, size_t workspace_bytes, void* stream) {
    REQUIRE(q && k && v && out, GDN_E_NULL, "gqa_prefill_attn: null pointer");
    REQUIRE(S >= 0 && pos >= 0 && (long long)pos + S < (1ll << 30), GDN_E_SHAPE, "gqa_prefill_attn: S=%d pos=%d", S, pos);
    REQUIRE(k_tok_stride > 0 && k_head_stride > 0 && v_tok_stride > 0 && v_head_stride > 0 && k_tok_stride % 8 == 0 && k_head_stride % 8 == 0 &&
                v_tok_stride % 8 == 0 && v_head_stride % 8 == 0,
            GDN_E_SHAPE, "gqa_prefill_attn: K / V strides must be positive multiples of 8 elements");
    REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out), GDN_E_ALIGN, "gqa_prefill_attn: tensors must be 16-byte aligned");
    if (S == 0) return GDN_OK;
    int* status = status_ptr();
    REQUIRE(status, GDN_E_LAUNCH, "gqa_prefill_attn: no CUDA device");
    REQUIRE(!workspace || aligned16(workspace), GDN_E_ALIGN, "gqa_prefill_attn: workspace must be 16-byte aligned");
    return launch_gqa_prefill(q, k, v, out, S, pos, k_tok_stride, k_head_stride, v_tok_stride, v_head_stride, workspace, workspace_bytes, status,
                              static_cast<cudaStream_t>(stream));
}

int gdn_conv_prep(const void* proj, long long row_stride, const void* conv_state, const void* conv_w, void* q, void* k, void* v, void* new_conv,
                  int S, void* stream) {
    REQUIRE(proj && conv_state && conv_w && q && k && v && new_conv, GDN_E_NULL, "gdn_conv_prep: null pointer");
    REQUIRE(S >= 0 && row_stride >= PW && row_stride % 4 == 0, GDN_E_SHAPE, "gdn_conv_prep: S=%d row_stride=%lld", S, row_stride);
    REQUIRE(((uintptr_t)proj | (uintptr_t)conv_state | (uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)new_conv) % 8 == 0, GDN_E_ALIGN,
            "gdn_conv_prep: tensors must be 8-byte aligned");
    typedef const __nv_bfloat16* cb; typedef __nv_bfloat16* b;
    return launch_conv_prep((cb)proj, row_stride, (cb)conv_state, (cb)conv_w, (b)q, (b)k, (b)v, (b)new_conv, S, static_cast<cudaStream_t>(stream));
}

int gdn_gated_norm(const void* y, const void* proj, long long row_stride, const float* gw, void* out, long long S, void* stream) {
    REQUIRE(y && proj && gw && out, GDN_E_NULL, "gdn_gated_norm: null pointer");
    REQUIRE(S >= 0 && row_stride >= PW && row_stride % 4 == 0, GDN_E_SHAPE, "gdn_gated_norm: S=%lld row_stride=%lld", S, row_stride);
    REQUIRE(((uintptr_t)y | (uintptr_t)proj | (uintptr_t)out) % 8 == 0, GDN_E_ALIGN, "gdn_gated_norm: tensors must be 8-byte aligned");
    return launch_gated_norm((const __nv_bfloat16*)y, (const __nv_bfloat16*)proj, row_stride, gw, (__nv_bfloat16*)out, S, static_cast<cudaStream_t>(stream));
}

int gdn_state_copy(void* dst, const void* src, int elem_size, long long n, long long d0, long long s0, int ny, long long dstride,
                   long long sstride, void* stream) {
    REQUIRE(dst && src, GDN_E_NULL, "gdn_state_copy: null pointer");
    REQUIRE(n >= 0 && d0 >= 0 && s0 >= 0 && ny >= 0, GDN_E_SHAPE, "gdn_state_copy: negative size");
    return launch_state_copy(dst, src, elem_size, n, d0, s0, ny, dstride, sstride, static_cast<cudaStream_t>(stream));
}

int gdn_hrec(void* hist, const void* rows, const int* slots, const int* pos, int B, int n_slots, int Lh, int H, void* stream) {
    REQUIRE(hist && rows && slots && pos, GDN_E_NULL, "gdn_hrec: null pointer");
    REQUIRE(B >= 0 && n_slots > 0 && Lh > 0 && H > 0, GDN_E_SHAPE, "gdn_hrec: B=%d n_slots=%d Lh=%d H=%d", B, n_slots, Lh, H);
    int* status = status_ptr();
    REQUIRE(status, GDN_E_LAUNCH, "gdn_hrec: no CUDA device");
    return launch_hrec(hist, rows, slots, pos, B, n_slots, Lh, H, status, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
