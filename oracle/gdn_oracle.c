/* C restatement (OpenMP) of the reference's GatedDeltaNet decode step and sequential rule.  TEST INFRASTRUCTURE ONLY:
 * it is the timed CPU baseline of the benchmark and a second checker; the shipped library never links it.
 *
 * Arithmetic follows, line by line, the reference's decode kernel qwen35/kernels.py:461-552 (conv window :476-484, q/k l2norm
 * :490-509, gates :511-515 with the bf16 helpers of qwen35/mslib.py:11-26, rule :518-533, window snapshot :528-541) and its
 * CPU statement of the rule bench/gdn_f64.py:48-56.  It is pinned against oracle/gdn_oracle.py (tests/test_oracle_c.py),
 * which in turn is pinned against outputs of the reference's own rec64.  Parallelism: OpenMP over (sequence, head).
 *
 * Build:  gcc -O3 -march=native -fopenmp -shared -fPIC -o oracle/_build/libgdn_oracle.so oracle/gdn_oracle.c -lm
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#define HV 16
#define DK 128
#define DV 128
#define KD 2048
#define CD 6144
#define PW 8224

static inline float bf(float x) {                       /* fp32 -> bf16 (nearest even) -> fp32 */
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7f800000u) == 0x7f800000u) return x;
    u = (u + 0x7fffu + ((u >> 16) & 1u)) & 0xffff0000u;
    memcpy(&x, &u, 4);
    return x;
}
static inline float ldbf(const uint16_t* p) { uint32_t u = (uint32_t)(*p) << 16; float f; memcpy(&f, &u, 4); return f; }
static inline uint16_t stbf(float x) { x = bf(x); uint32_t u; memcpy(&u, &x, 4); return (uint16_t)(u >> 16); }

static inline float sigmoid_bf16(float x) {              /* mslib.py:16-20 */
    float y = bf(1.0f / bf(1.0f + bf(expf(fabsf(x)))));
    return x < 0.0f ? y : bf(1.0f - y);
}
static inline float silu_bf16(float x) { return bf(x * sigmoid_bf16(x)); }
static inline float softplus_bf16(float x) { return bf(fmaxf(x, 0.0f) + bf(log1pf(bf(expf(-fabsf(x)))))); }

/* One decode step for B sequences, in place (the layout of deltanet_b, qwen35/batch.py:36-135):
 *   proj bf16 [B, PW]; conv_pool bf16 [n_slots*2, 3, CD]; conv_w bf16 [CD*4]; ssm_pool fp32 [n_slots, HV, DV, DK];
 *   slots, pos int32 [B]; y bf16 [B, HV*DV]. */
void oracle_deltanet_b(const uint16_t* proj, uint16_t* conv_pool, const uint16_t* conv_w, const float* A_log, const float* dt_bias,
                       float* ssm_pool, const int* slots, const int* pos, uint16_t* y, int B) {
    const float inv_scale = 0.08838834764831845f;
    const float e2 = 1e-6f * inv_scale * inv_scale;
    const float sc_q = bf(inv_scale * inv_scale), sc_k = bf(inv_scale);
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; b++) {
        for (int hv = 0; hv < HV; hv++) {
            const size_t slot = (size_t)slots[b];
            const unsigned par = (unsigned)pos[b] & 1u;
            const uint16_t* cs_in = conv_pool + (slot * 2 + par) * 3 * CD;
            uint16_t* cs_out = conv_pool + (slot * 2 + (par ^ 1u)) * 3 * CD;
            const uint16_t* pj = proj + (size_t)b * PW;
            float* S = ssm_pool + (slot * HV + hv) * DV * DK;
            float q[DK], k[DK], v[DV];
            float qs = 0.f, ks = 0.f;
            for (int g = 0; g < 3; g++) {
                for (int c = 0; c < DK; c++) {
                    const int ch = g * KD + hv * DK + c;
                    float o = ldbf(cs_in + ch) * ldbf(conv_w + ch * 4);
                    o += ldbf(cs_in + CD + ch) * ldbf(conv_w + ch * 4 + 1);
                    o += ldbf(cs_in + 2 * CD + ch) * ldbf(conv_w + ch * 4 + 2);
                    o += ldbf(pj + ch) * ldbf(conv_w + ch * 4 + 3);
                    o = silu_bf16(bf(o));
                    if (g == 0) { q[c] = o; qs += o * o; } else if (g == 1) { k[c] = o; ks += o * o; } else v[c] = o;
                    cs_out[ch] = cs_in[CD + ch];
                    cs_out[CD + ch] = cs_in[2 * CD + ch];
                    cs_out[2 * CD + ch] = pj[ch];
                }
            }
            const float qr = 1.0f / sqrtf(qs / (float)DK + e2), kr = 1.0f / sqrtf(ks / (float)DK + e2);
            for (int c = 0; c < DK; c++) { q[c] = bf(bf(q[c] * qr) * sc_q); k[c] = bf(bf(k[c] * kr) * sc_k); }
            const float av = bf(ldbf(pj + CD + KD + HV + hv) + dt_bias[hv]);
            const float g = expf(-expf(A_log[hv]) * softplus_bf16(av));
            const float beta = sigmoid_bf16(ldbf(pj + CD + KD + hv));
            for (int r = 0; r < DV; r++) {
                float* s = S + (size_t)r * DK;
                float kvm = 0.f;
                for (int c = 0; c < DK; c++) { s[c] *= g; kvm += s[c] * k[c]; }
                const float delta = (v[r] - kvm) * beta;
                float yv = 0.f;
                for (int c = 0; c < DK; c++) { s[c] += k[c] * delta; yv += s[c] * q[c]; }
                y[(size_t)b * HV * DV + hv * DV + r] = stbf(yv);
            }
        }
    }
}

/* Sequential rule over T tokens (gated_delta_update's kernel; bench/gdn_f64.py:48-56 in fp32):
 *   q, k, v bf16 [B,T,H,128]; g, beta fp32 [B,T,H]; S fp32 [B,H,128,128] in/out; y bf16 [B,T,H,128]. */
void oracle_gated_delta_rule(const uint16_t* q, const uint16_t* k, const uint16_t* v, const float* g, const float* beta, float* S,
                             uint16_t* y, int B, int T, int H) {
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int b = 0; b < B; b++) {
        for (int h = 0; h < H; h++) {
            float* Sh = S + ((size_t)b * H + h) * DV * DK;
            for (int t = 0; t < T; t++) {
                const size_t o = (((size_t)b * T + t) * H + h) * DK;
                float kf[DK], qf[DK];
                for (int c = 0; c < DK; c++) { kf[c] = ldbf(k + o + c); qf[c] = ldbf(q + o + c); }
                const float gt = g[((size_t)b * T + t) * H + h], bt = beta[((size_t)b * T + t) * H + h];
                for (int r = 0; r < DV; r++) {
                    float* s = Sh + (size_t)r * DK;
                    float kvm = 0.f;
                    for (int c = 0; c < DK; c++) { s[c] *= gt; kvm += s[c] * kf[c]; }
                    const float delta = (ldbf(v + o + r) - kvm) * bt;
                    float yv = 0.f;
                    for (int c = 0; c < DK; c++) { s[c] += kf[c] * delta; yv += s[c] * qf[c]; }
                    y[o + r] = stbf(yv);
                }
            }
        }
    }
}

/* GQA decode attention for one query row over contiguous K/V (qwen35/batch.py:141-227), fp32:
 *   q bf16 [H=8, 256]; K, V bf16 [KV=2, n, 256]; o bf16 [8, 256]. */
void oracle_attn_row(const uint16_t* q, const uint16_t* K, const uint16_t* V, uint16_t* o, int n) {
#pragma omp parallel for schedule(static)
    for (int h = 0; h < 8; h++) {
        const int kv = h / 4;
        float m = -INFINITY, l = 0.f, acc[256];
        for (int d = 0; d < 256; d++) acc[d] = 0.f;
        for (int i = 0; i < n; i++) {
            const uint16_t* kr = K + ((size_t)kv * n + i) * 256;
            const uint16_t* vr = V + ((size_t)kv * n + i) * 256;
            float s = 0.f;
            for (int d = 0; d < 256; d++) s += 0.0625f * ldbf(q + h * 256 + d) * ldbf(kr + d);
            const float mn = fmaxf(m, s), f = expf(m - mn), p = expf(s - mn);
            l = l * f + p;
            for (int d = 0; d < 256; d++) acc[d] = acc[d] * f + p * ldbf(vr + d);
            m = mn;
        }
        for (int d = 0; d < 256; d++) o[h * 256 + d] = stbf(l == 0.f ? acc[d] : acc[d] / l);
    }
}

int oracle_max_threads(void);
#ifdef _OPENMP
#include <omp.h>
int oracle_max_threads(void) { return omp_get_max_threads(); }
#else
int oracle_max_threads(void) { return 1; }
#endif
