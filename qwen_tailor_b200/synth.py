"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

They stand in for real Qwen3.5-0.8B activations (the weights are not available offline).  Common to every case:
H = 16 heads, d_k = d_v = 128; q, k, v bf16 ~ N(0, 1) with q, k L2-normalised per head (q additionally scaled by
128^-1/2); beta = sigmoid(b), b ~ N(0, 1); log-decay = -exp(A_log) * softplus(a + dt_bias) with A_log ~ U(0, ln 16),
a ~ N(0, 1), dt_bias ~ N(0, 0.1).  Everything is generated with numpy's PCG64 so the same seed gives the same arrays on
every host; arrays that are bf16 on the device are returned as fp32 arrays holding bf16-exact values.
"""
from __future__ import annotations

import math

import numpy as np

HV, DK, DV, KD, CD, PW = 16, 128, 128, 2048, 6144, 8224
N_GDN_LAYERS, N_ATTN_LAYERS = 18, 6
ATT_H, ATT_KV, ATT_D = 8, 2, 256


def bf16r(x):
    """Round an fp32 array to the nearest bf16 value (ties to even), keeping fp32 storage."""
    a = np.ascontiguousarray(np.asarray(x, dtype=np.float32))
    u = a.view(np.uint32)
    r = ((u >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
    return ((u + r) & np.uint32(0xFFFF0000)).view(np.float32).reshape(a.shape)


def to_torch_bf16(x, device=None):
    """fp32 numpy array of bf16-exact values -> torch.bfloat16 tensor (exact)."""
    import torch
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(device=device, dtype=torch.bfloat16)


def layer_params(rng):
    """A_log [16] fp32 ~ U(0, ln 16), dt_bias [16] ~ N(0, 0.1) (bf16-exact)."""
    A_log = rng.uniform(0.0, math.log(16.0), HV).astype(np.float32)
    dt_bias = bf16r(rng.normal(0.0, 0.1, HV))
    return A_log, dt_bias


def _unit(x):
    n = np.sqrt((x.astype(np.float64) ** 2).sum(-1, keepdims=True))
    return (x / np.maximum(n, 1e-12)).astype(np.float32)


def gdn_tokens(rng, T, lead=()):
    """q, k, v [*lead, T, 16, 128] (normalised as the rule expects), a, b [*lead, T, 16]."""
    shp = tuple(lead) + (T, HV, DK)
    q = bf16r(_unit(bf16r(rng.standard_normal(shp))) * np.float32(DK ** -0.5))
    k = bf16r(_unit(bf16r(rng.standard_normal(shp))))
    v = bf16r(rng.standard_normal(tuple(lead) + (T, HV, DV)))
    a = bf16r(rng.standard_normal(tuple(lead) + (T, HV)))
    b = bf16r(rng.standard_normal(tuple(lead) + (T, HV)))
    return q, k, v, a, b


def config1(seed=0, T=256):
    """Single layer, full-sequence forward: B=1, T=256, zero initial state."""
    rng = np.random.default_rng(seed)
    A_log, dt_bias = layer_params(rng)
    q, k, v, a, b = gdn_tokens(rng, T, lead=(1,))
    return dict(q=q, k=k, v=v, a=a, b=b, A_log=A_log, dt_bias=dt_bias, state=np.zeros((1, HV, DV, DK), np.float32))


def conv_weights(rng):
    """Depthwise conv taps [6144*4] (flat ch*4+tap, tap 3 = current token), bf16-exact, ~N(0, 0.5)."""
    return bf16r(rng.standard_normal(CD * 4) * 0.5)


def config2(B, seed=1, M=1):
    """Recurrent decode step: proj rows [B*M, 8224] (mixed qkv | z | b | a), conv window [B, 3, 6144], state [B,16,128,128] ~ N(0, 0.02)."""
    rng = np.random.default_rng(seed)
    A_log, dt_bias = layer_params(rng)
    conv_w = conv_weights(rng)
    proj = bf16r(rng.standard_normal((B * M, PW)))
    conv = bf16r(rng.standard_normal((B, 3, CD)))
    state = (rng.standard_normal((B, HV, DV, DK)) * 0.02).astype(np.float32)
    return dict(proj=proj, conv=conv, conv_w=conv_w, A_log=A_log, dt_bias=dt_bias, state=state)


def config3_layer(layer, T):
    """One of the 18 independent layers of the long-prefill case (seed 100 + layer), zero initial state."""
    rng = np.random.default_rng(100 + layer)
    A_log, dt_bias = layer_params(rng)
    q, k, v, a, b = gdn_tokens(rng, T)
    return dict(q=q, k=k, v=v, a=a, b=b, A_log=A_log, dt_bias=dt_bias)


def config4_lengths(seed=7, n_seq=16, lo=128, hi=4096):
    """Ragged batch: lengths ~ U[lo, hi]; every second sequence resumes from a cached prefix whose length is a multiple of 64.

    Returns (lengths [n], prefix [n]) where prefix[i] = 0 for sequences that start from scratch."""
    rng = np.random.default_rng(seed)
    lengths = rng.integers(lo, hi + 1, n_seq).astype(np.int64)
    prefix = np.zeros(n_seq, np.int64)
    for i in range(1, n_seq, 2):
        prefix[i] = 64 * int(rng.integers(1, max(2, lengths[i] // 64)))
        prefix[i] = min(prefix[i], (lengths[i] - 1) // 64 * 64)
    return lengths, prefix


def config4(seed=7, n_seq=16, lo=128, hi=4096):
    """Packed varlen prefill with prefix-cache resume.  Only the suffix of a resuming sequence is computed."""
    lengths, prefix = config4_lengths(seed, n_seq, lo, hi)
    rng = np.random.default_rng(seed + 1)
    A_log, dt_bias = layer_params(rng)
    suffix = lengths - prefix
    cu = np.zeros(n_seq + 1, np.int32)
    cu[1:] = np.cumsum(suffix)
    q, k, v, a, b = gdn_tokens(rng, int(cu[-1]))
    init = (rng.standard_normal((n_seq, HV, DV, DK)) * 0.02).astype(np.float32)
    init[prefix == 0] = 0.0
    return dict(q=q, k=k, v=v, a=a, b=b, A_log=A_log, dt_bias=dt_bias, cu_seqlens=cu, init_state=init,
                has_init=(prefix > 0), lengths=lengths, prefix=prefix)


def config5_shapes(seed=11, B=16, K=4, lo=1024, hi=8192):
    """Speculative verify step: context lengths ~ U[lo, hi] and accept lengths ~ U{0..K}."""
    rng = np.random.default_rng(seed)
    ctx = rng.integers(lo, hi + 1, B).astype(np.int32)
    accept = rng.integers(0, K + 1, B).astype(np.int32)
    return ctx, accept


def attn_case(rng, ctx, M, page_size):
    """Paged GQA decode inputs for sequences with the given context lengths.

    Returns q [B*M, 8, 256], k_new / v_new [B*M, 2, 256], pages K / V [n_pages, 2, page_size, 256] (entries ~ N(0,1)),
    block_table [B, max_pages] int32 (pages handed out in a shuffled order)."""
    ctx = np.asarray(ctx, np.int64)
    B = len(ctx)
    need = (ctx + M + page_size - 1) // page_size
    max_pages = int(need.max())
    n_pages = int(need.sum()) + 1
    order = rng.permutation(n_pages - 1) + 1                  # page 0 stays unused (catches stray writes)
    table = np.zeros((B, max_pages), np.int32)
    o = 0
    for i in range(B):
        table[i, :need[i]] = order[o:o + need[i]]
        o += need[i]
    Kp = bf16r(rng.standard_normal((n_pages, ATT_KV, page_size, ATT_D)))
    Vp = bf16r(rng.standard_normal((n_pages, ATT_KV, page_size, ATT_D)))
    q = bf16r(rng.standard_normal((B * M, ATT_H, ATT_D)))
    kn = bf16r(rng.standard_normal((B * M, ATT_KV, ATT_D)))
    vn = bf16r(rng.standard_normal((B * M, ATT_KV, ATT_D)))
    return dict(q=q, k_new=kn, v_new=vn, k_pages=Kp, v_pages=Vp, block_table=table, ctx_len=ctx.astype(np.int32))
