"""CPU restatement (numpy) of the reference's GatedDeltaNet / GQA-decode arithmetic.  TEST INFRASTRUCTURE ONLY.

This module is the checker the CUDA kernels are compared with.  Nothing in the shipped package imports it; only the test
suite, the smoke check and the CPU-baseline leg of the benchmark do.

Parity status: the reference publishes no operator-level golden vectors and its runtime (MLX / Metal) cannot run on a
Linux host.  What *can* be executed from the reference is its own CPU statement of the rule, ``rec64`` in
``bench/gdn_f64.py:48-56`` (pure numpy); ``tests/golden/make_golden.py`` runs that function unmodified on seeded inputs and
stores its outputs, and ``tests/test_oracle.py`` pins ``gated_delta_rule`` below against those vectors.  Everything that
lives in the reference's Metal kernels only (gate rounding points, the conv window, snapshots, attention) is restated from
the cited source lines and is **parity unpinned**: no executable reference output exists for it on this platform.

Every function cites the reference lines it follows (paths relative to the reference project root).

Two precisions are offered everywhere: ``dtype=np.float64`` is the accuracy truth (gate rounding points kept, because they
are part of the function's definition; the recurrence itself in fp64), ``dtype=np.float32`` follows the reference kernels'
fp32 arithmetic and is what the timed CPU baseline runs.
"""
from __future__ import annotations

import numpy as np

HV, DK, DV, KD, CD, PW = 16, 128, 128, 2048, 6144, 8224      # qwen35/batch.py:29, qwen35/kernels.py:466


# ---------------------------------------------------------------------------------------------------------------------
# bf16 helpers
# ---------------------------------------------------------------------------------------------------------------------
def bf16_round(x):
    """fp32 -> bf16 (round to nearest even) -> fp32; the reference's ``BF(v)`` macro (qwen35/kernels.py:22-24)."""
    a = np.ascontiguousarray(np.asarray(x, dtype=np.float32))
    u = a.view(np.uint32)
    r = ((u >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
    out = ((u + r) & np.uint32(0xFFFF0000)).view(np.float32)
    return np.where(np.isfinite(a), out, a).astype(np.float32).reshape(a.shape)


def bf16_bits(x):
    """fp32 array holding bf16-exact values -> uint16 bit patterns."""
    return (np.ascontiguousarray(np.asarray(x, np.float32)).view(np.uint32) >> np.uint32(16)).astype(np.uint16)


def bf16_from_bits(u):
    return (np.asarray(u, np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def sigmoid_bf16(x):
    """mx.sigmoid on a bf16 array: 1/(1+exp(|x|)) rounded after every op, mirrored for x >= 0 (qwen35/mslib.py:16-20)."""
    x = np.asarray(x, np.float32)
    with np.errstate(over="ignore"):
        y = bf16_round(1.0 / bf16_round(1.0 + bf16_round(np.exp(np.abs(x)))))
    return np.where(x < 0, y, bf16_round(1.0 - y)).astype(np.float32)


def silu_bf16(x):
    """nn.silu on bf16 = x * sigmoid(x), product rounded (qwen35/mslib.py:21-22)."""
    x = np.asarray(x, np.float32)
    return bf16_round(x * sigmoid_bf16(x))


def softplus_bf16(x):
    """nn.softplus on bf16 = max(x,0) + log1p(exp(-|x|)) with bf16 rounding of exp, log1p and the sum (qwen35/mslib.py:23-26)."""
    x = np.asarray(x, np.float32)
    e = bf16_round(np.exp(-np.abs(x)))
    return bf16_round(np.maximum(x, 0.0) + bf16_round(np.log1p(e.astype(np.float64)).astype(np.float32)))


# ---------------------------------------------------------------------------------------------------------------------
# gates and q/k normalisation
# ---------------------------------------------------------------------------------------------------------------------
def log_decay(A_log, a, dt_bias):
    """log of the per-token decay: -exp(A_log) * softplus_bf16(bf16(a + dt_bias)).

    qwen35/gated_delta.py:16-18 (compute_g), rounding points qwen35/kernels.py:511-513 and bench/gdn_f64.py:39-45.
    A_log, dt_bias: [H]; a: [..., H] (bf16-exact values).  Returns fp32 [..., H]."""
    av = bf16_round(np.asarray(a, np.float32) + np.asarray(dt_bias, np.float32))
    sp = softplus_bf16(av)
    return (-np.exp(np.asarray(A_log, np.float32)) * sp).astype(np.float32)


def compute_g(A_log, a, dt_bias):
    """decay g = exp(log_decay) in fp32 (qwen35/gated_delta.py:16-18)."""
    return np.exp(log_decay(A_log, a, dt_bias)).astype(np.float32)


def beta_gate(b):
    """beta = sigmoid(b) evaluated in bf16 (qwen35/gated_delta.py:158, qwen35/kernels.py:514-515)."""
    return sigmoid_bf16(b)


def normalize_qk(q, k, inv_scale=DK ** -0.5, eps=1e-6):
    """q <- l2norm(q) * inv_scale^2, k <- l2norm(k) * inv_scale, with the reference's rounding points.

    qwen35/gated_delta.py:21-30 (rms_norm with eps * inv_scale^2, then a bf16 scalar multiply) and the kernel form
    qwen35/kernels.py:490-509: ``BF(BF(x * rsqrt(mean(x^2) + e2)) * BF(scale))``.  q, k: [..., D] bf16-exact values."""
    q = np.asarray(q, np.float32)
    k = np.asarray(k, np.float32)
    e2 = np.float32(eps) * np.float32(inv_scale) * np.float32(inv_scale)
    sc_q = bf16_round(np.float32(inv_scale) * np.float32(inv_scale))
    sc_k = bf16_round(np.float32(inv_scale))

    def one(x, sc):
        ms = (x.astype(np.float64) ** 2).sum(-1, keepdims=True) / x.shape[-1]
        r = (1.0 / np.sqrt(ms + e2)).astype(np.float32)
        return bf16_round(bf16_round(x * r) * sc)
    return one(q, sc_q), one(k, sc_k)


# ---------------------------------------------------------------------------------------------------------------------
# the sequential gated delta rule
# ---------------------------------------------------------------------------------------------------------------------
def gated_delta_rule(q, k, v, g, beta, S0, dtype=np.float64):
    """Sequential rule over T tokens for one sequence.

    bench/gdn_f64.py:48-56 (rec64) and the kernel body qwen35/gated_delta.py:75-126:
        S <- g_t S;  kv = S k_t;  d = (v_t - kv) beta_t;  S <- S + d k_t^T;  y_t = S q_t
    q, k: [T, H, Dk]; v: [T, H, Dv]; g, beta: [T, H]; S0: [H, Dv, Dk].  Returns (y [T, H, Dv], S [H, Dv, Dk]) in ``dtype``."""
    q, k, v, g, beta = (np.asarray(x, dtype) for x in (q, k, v, g, beta))
    S = np.array(S0, dtype=dtype, copy=True)
    T = q.shape[0]
    ys = np.zeros((T,) + v.shape[1:], dtype)
    for t in range(T):
        S *= g[t][:, None, None]
        kv = np.einsum("hvk,hk->hv", S, k[t])
        d = (v[t] - kv) * beta[t][:, None]
        S += d[:, :, None] * k[t][:, None, :]
        ys[t] = np.einsum("hvk,hk->hv", S, q[t])
    return ys, S


def gated_delta_update(q, k, v, a, b, A_log, dt_bias, state=None, dtype=np.float64):
    """Ops-level entry point (qwen35/gated_delta.py:143-174): gates from (a, b), then the rule, batched.

    q, k: [B, T, Hk, Dk] (already normalised); v: [B, T, Hv, Dv]; a, b: [B, T, Hv]; state [B, Hv, Dv, Dk] or None (zeros).
    Returns (y [B, T, Hv, Dv] rounded to bf16 as fp32 values, y unrounded in ``dtype``, state)."""
    q, k, v = (np.asarray(x, np.float32) for x in (q, k, v))
    B, T, Hk, Dk = k.shape
    Hv, Dv = v.shape[2:]
    if Dk != 128 or Dv % 8:
        raise ValueError("only Dk=128, Dv%8==0 is supported")          # qwen35/gated_delta.py:164-166
    g = compute_g(A_log, a, dt_bias)
    beta = beta_gate(b)
    if state is None:
        state = np.zeros((B, Hv, Dv, Dk), np.float32)
    ys, Ss = [], []
    for i in range(B):
        y, S = gated_delta_rule(q[i], k[i], v[i], g[i], beta[i], state[i], dtype)
        ys.append(y)
        Ss.append(S)
    y = np.stack(ys)
    return bf16_round(y.astype(np.float32)), y, np.stack(Ss)


def chunked_rule(q, k, v, lg, beta, S0, C=64, dtype=np.float64):
    """The chunked WY/UT form of the rule (qwen35/gdn_nax.py:3-10), chunk of C tokens, one sequence.

        L = strict_lower(beta_i G_ij (K K^T)_ij), G_ij = exp(Lc_i - Lc_j), Lc = inclusive cumulative log-decay in the chunk
        T = (I + L)^-1, Tb = T diag(beta);  D = Tb (V - gamma * (K S0^T)), gamma_i = exp(Lc_i)
        Y = gamma * (Q S0^T) + A D, A = lower_incl(G * Q K^T);  S1 = gamma_C S0 + D^T diag(gamma_C / gamma) K
    Decay factors are formed from differences of Lc and masked before the exp (qwen35/gdn_nax.py:100-103,125).
    A partial last chunk behaves as if its missing rows were zero (qwen35/gdn_nax.py:55-60).  lg: log-decay [T, H]."""
    q, k, v, lg, beta = (np.asarray(x, dtype) for x in (q, k, v, lg, beta))
    S = np.array(S0, dtype=dtype, copy=True)
    T, H = lg.shape
    y = np.zeros((T, H, v.shape[2]), dtype)
    for t0 in range(0, T, C):
        n = min(C, T - t0)
        for h in range(H):
            K, Q, V = k[t0:t0 + n, h], q[t0:t0 + n, h], v[t0:t0 + n, h]
            Lc = np.cumsum(lg[t0:t0 + n, h])
            diff = Lc[:, None] - Lc[None, :]
            low = np.tril(np.ones((n, n), bool))
            G = np.where(low, np.exp(np.where(low, diff, 0.0)), 0.0)
            Lm = np.tril(beta[t0:t0 + n, h][:, None] * G * (K @ K.T), -1)
            Tm = np.linalg.solve(np.eye(n, dtype=dtype) + Lm, np.eye(n, dtype=dtype))
            Tb = Tm * beta[t0:t0 + n, h][None, :]
            gam = np.exp(Lc)
            D = Tb @ (V - gam[:, None] * (K @ S[h].T))
            A = G * (Q @ K.T)
            y[t0:t0 + n, h] = gam[:, None] * (Q @ S[h].T) + A @ D
            dec = np.exp(Lc[-1] - Lc)
            S[h] = gam[-1] * S[h] + (D * dec[:, None]).T @ K
    return y, S


# ---------------------------------------------------------------------------------------------------------------------
# decode / speculative verify (conv window + gates + rule + snapshots)
# ---------------------------------------------------------------------------------------------------------------------
def deltanet(proj, conv_win, conv_w, A_log, dt_bias, S0, dtype=np.float32):
    """M chained tokens of one sequence through conv(4 taps)+silu, q/k l2norm, gates and the rule, with a state snapshot
    and a conv-window snapshot after every token.  qwen35/kernels.py:461-552 (same arithmetic: qwen35/batch.py:57-119,
    qwen35/batch_spec.py:68-133).

    proj [M, 8224] (qkv 6144 | z 2048 | b 16 | a 16), conv_win [3, 6144] (the last 3 raw mixed-qkv rows, oldest first),
    conv_w [6144*4] flat ``ch*4+tap`` (tap 3 = current token), S0 [16, 128, 128].  All bf16-exact fp32 values except S0.
    Returns (y bf16-rounded [M, 2048], y unrounded, conv snapshots [M, 3, 6144], state snapshots [M, 16, 128, 128])."""
    proj = np.asarray(proj, np.float32)
    M = proj.shape[0]
    w = np.asarray(conv_w, np.float32).reshape(CD, 4)
    rows = np.concatenate([np.asarray(conv_win, np.float32).reshape(3, CD), proj[:, :CD]], axis=0)    # index t+3  (kernels.py:477-479)
    A_log = np.asarray(A_log, np.float32)
    dt_bias = np.asarray(dt_bias, np.float32)
    S = np.array(S0, dtype=dtype, copy=True)
    ys, yu, cs, st = [], [], [], []
    for j in range(M):
        acc = rows[j] * w[:, 0]                                                  # fp32, left to right (kernels.py:480-484)
        acc = acc + rows[j + 1] * w[:, 1]
        acc = acc + rows[j + 2] * w[:, 2]
        acc = acc + rows[j + 3] * w[:, 3]
        c = silu_bf16(bf16_round(acc))
        qn, kn = normalize_qk(c[:KD].reshape(HV, DK), c[KD:2 * KD].reshape(HV, DK))     # kernels.py:490-509
        vv = c[2 * KD:].reshape(HV, DV)
        g = compute_g(A_log, proj[j, CD + KD + HV:CD + KD + 2 * HV], dt_bias)     # a at 8208.. (kernels.py:511-513)
        beta = beta_gate(proj[j, CD + KD:CD + KD + HV])                          # b at 8192.. (kernels.py:514-515)
        y, S = gated_delta_rule(qn[None], kn[None], vv[None], g[None], beta[None], S, dtype)      # kernels.py:518-533
        yu.append(y[0].reshape(-1))
        ys.append(bf16_round(y[0].reshape(-1).astype(np.float32)))
        cs.append(rows[j + 1:j + 4].copy())                                       # kernels.py:528-541
        st.append(S.copy())
    return np.stack(ys), np.stack(yu), np.stack(cs), np.stack(st)


# ---------------------------------------------------------------------------------------------------------------------
# GQA decode attention over a slot pool / paged cache
# ---------------------------------------------------------------------------------------------------------------------
def attn_rows(q, k_new, v_new, k_ctx, v_ctx, dtype=np.float64):
    """Decode attention of M chained query rows of ONE sequence.  qwen35/batch.py:141-227.

    q [M, H, D]; k_new, v_new [M, KV, D] (the rows appended by this call); k_ctx, v_ctx [KV, ctx, D] (rows already cached).
    Row j attends the ctx cached keys and new rows 0..j; softmax scale D^-1/2 is applied to q (0.0625 for D=256,
    batch.py:176).  Returns o [M, H, D] in ``dtype`` (unrounded)."""
    q, k_new, v_new, k_ctx, v_ctx = (np.asarray(x, dtype) for x in (q, k_new, v_new, k_ctx, v_ctx))
    M, H, D = q.shape
    KV = k_new.shape[1]
    out = np.zeros((M, H, D), dtype)
    for j in range(M):
        for h in range(H):
            kv = h // (H // KV)
            keys = np.concatenate([k_ctx[kv], k_new[:j + 1, kv]], axis=0)
            vals = np.concatenate([v_ctx[kv], v_new[:j + 1, kv]], axis=0)
            s = keys @ (q[j, h] * dtype(D ** -0.5))
            p = np.exp(s - s.max())
            out[j, h] = (p @ vals) / p.sum()
    return out


def prefill_attention(q, K, V, pos=0, dtype=np.float64):
    """Causal attention of a prefill chunk: the scaled_dot_product_attention call of qwen35/model.py:165 (scale D^-1/2, causal mask,
    GQA: query head h reads KV head h // (H // KV)).

    q [S, H, D]: queries at positions pos .. pos + S - 1; K, V [KV, T, D] with T >= pos + S.  Returns o [S, H, D] in ``dtype`` (unrounded)."""
    q, K, V = (np.asarray(x, dtype) for x in (q, K, V))
    S, H, D = q.shape
    KV = K.shape[0]
    out = np.zeros((S, H, D), dtype)
    for h in range(H):
        kv = h // (H // KV)
        s = (q[:, h] * dtype(D ** -0.5)) @ K[kv, :pos + S].T                      # [S, pos + S]
        s = np.where(np.arange(pos + S)[None, :] <= (pos + np.arange(S))[:, None], s, -np.inf)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        out[:, h] = (p @ V[kv, :pos + S]) / p.sum(axis=1, keepdims=True)
    return out


def qkv_prep(qkv, q_norm, k_norm, row_pos, eps=1e-6, theta=1e7, rope_dim=64):
    """Attention glue in front of the decode attention (qwen35/fast.py:70-78, qwen35/model.py:148-161): split a qkv row into
    8 x (q 256 | gate 256), k 2 x 256, v 2 x 256; rms_norm q and k over 256 with weights; rotate dims [0, 64) of q and k
    (half-split pairs i, i + 32; angle pos * theta^(-i/32)).  One bf16 rounding after the norm and one after the rotation,
    as two MLX ops give.  Returns (q [R,8,256], gate [R,2048], k [R,2,256], v [R,2,256]) as bf16-exact fp32."""
    qkv = np.asarray(qkv, np.float32)
    R = qkv.shape[0]
    qg = qkv[:, :4096].reshape(R, 8, 512)
    q, gate = qg[:, :, :256], qg[:, :, 256:].reshape(R, 2048)
    k = qkv[:, 4096:4608].reshape(R, 2, 256)
    v = qkv[:, 4608:5120].reshape(R, 2, 256)

    def norm(x, w):
        ms = (x.astype(np.float64) ** 2).mean(-1, keepdims=True)
        return bf16_round((x / np.sqrt(ms + eps) * np.asarray(w, np.float64)).astype(np.float32))

    def rope(x):
        half = rope_dim // 2
        ang = np.asarray(row_pos, np.float64)[:, None, None] * theta ** (-np.arange(half) / half)[None, None, :]
        x1, x2 = x[..., :half].astype(np.float64), x[..., half:rope_dim].astype(np.float64)
        out = x.copy()
        out[..., :half] = bf16_round((x1 * np.cos(ang) - x2 * np.sin(ang)).astype(np.float32))
        out[..., half:rope_dim] = bf16_round((x1 * np.sin(ang) + x2 * np.cos(ang)).astype(np.float32))
        return out
    return rope(norm(q, q_norm)), gate.copy(), rope(norm(k, k_norm)), v.copy()


def gate_out(o, gate):
    """o * sigmoid(gate) on bf16 arrays (qwen35/fast.py:84): sigmoid evaluated op by op in bf16, product rounded."""
    return bf16_round(np.asarray(o, np.float32) * sigmoid_bf16(gate))


def conv_prep(proj, conv_state, conv_w):
    """Prefill conv + silu + q/k l2norm over S tokens (qwen35/prefill.py:96-134,160-238) and the new window (:262-263).
    proj [S, 8224], conv_state [3, 6144], conv_w [6144*4].  Returns (q, k, v [S,16,128], new_conv [3,6144])."""
    proj = np.asarray(proj, np.float32)
    S = proj.shape[0]
    w = np.asarray(conv_w, np.float32).reshape(CD, 4)
    rows = np.concatenate([np.asarray(conv_state, np.float32).reshape(3, CD), proj[:, :CD]], axis=0)
    acc = rows[0:S] * w[:, 0]
    acc = acc + rows[1:S + 1] * w[:, 1]
    acc = acc + rows[2:S + 2] * w[:, 2]
    acc = acc + rows[3:S + 3] * w[:, 3]
    c = silu_bf16(bf16_round(acc))
    q, k = normalize_qk(c[:, :KD].reshape(S, HV, DK), c[:, KD:2 * KD].reshape(S, HV, DK))
    return q, k, c[:, 2 * KD:].reshape(S, HV, DV), rows[S:S + 3].copy()


def gated_norm(y, proj, gw):
    """silu(z) * gw * y * rsqrt(mean(y^2) + 1e-6) per (token, head), one rounding at the end (qwen35/prefill.py:137-157)."""
    y = np.asarray(y, np.float64).reshape(-1, HV, DV)
    z = np.asarray(proj, np.float64)[:, CD:CD + HV * DV].reshape(-1, HV, DV)
    inv = 1.0 / np.sqrt((y ** 2).mean(-1, keepdims=True) + 1e-6)
    out = z / (1.0 + np.exp(-z)) * (np.asarray(gw, np.float64)[None, None, :] * (y * inv))
    return bf16_round(out.astype(np.float32)).reshape(-1, HV * DV)


# ---------------------------------------------------------------------------------------------------------------------
# speculative acceptance (integer work: bit-exact contract)
# ---------------------------------------------------------------------------------------------------------------------
def accept_length(toks, ids):
    """n_new = sum(cumprod(toks[:, 1:] == ids[:, :k])) per row (qwen35/spec.py:60-61, qwen35/batch_spec.py:380-381)."""
    toks = np.asarray(toks)
    ids = np.asarray(ids)
    k = toks.shape[1] - 1
    eq = (toks[:, 1:] == ids[:, :k]).astype(np.int32)
    return np.cumprod(eq, axis=1).sum(axis=1).astype(np.int32)


# ---------------------------------------------------------------------------------------------------------------------
# error measures used by every parity test
# ---------------------------------------------------------------------------------------------------------------------
def max_err_scaled(x, ref):
    """max|x - ref| / max|ref| (the reference's own normalisation, tests/kernels.py:8-12)."""
    x = np.asarray(x, np.float64)
    ref = np.asarray(ref, np.float64)
    return float(np.abs(x - ref).max() / max(np.abs(ref).max(), 1e-30))


def rel_l2(x, ref):
    """||x - ref|| / ||ref|| (bench/gdn_nax.py:17-22)."""
    x = np.asarray(x, np.float64).reshape(-1)
    ref = np.asarray(ref, np.float64).reshape(-1)
    return float(np.linalg.norm(x - ref) / max(np.linalg.norm(ref), 1e-30))


def bf16_ulp_distance(x, ref):
    """Elementwise distance in bf16 units-in-the-last-place of ``ref`` between two bf16-exact arrays."""
    x = np.asarray(x, np.float32)
    ref = np.asarray(ref, np.float32)
    ulp = np.exp2(np.floor(np.log2(np.maximum(np.abs(ref), 1e-30))) - 7)
    return np.abs(x.astype(np.float64) - ref) / ulp
