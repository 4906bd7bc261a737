"""CPU tests of the oracle: pinned against the golden vectors produced by the reference's own rec64, and checked for the
algebraic identities the CUDA kernels rely on."""
from pathlib import Path

import numpy as np
import pytest

from oracle import gdn_oracle as orc
from qwen_tailor_b200 import synth

GOLD = Path(__file__).parent / "golden" / "rec64_kat.npz"


def _warm_state(scale):
    h = np.arange(16)[:, None, None]
    v = np.arange(128)[None, :, None]
    k = np.arange(128)[None, None, :]
    return (scale * np.cos(0.37 * h + 0.11 * v + 0.05 * k + 0.013 * v * k)).astype(np.float32)


@pytest.mark.parametrize("name", ["zero_state", "warm_state"])
def test_rule_matches_reference_rec64(name):
    """gated_delta_rule == the reference's rec64 (bench/gdn_f64.py:48-56) on the stored known-answer vectors."""
    z = np.load(GOLD)
    q, k, v = (orc.bf16_from_bits(z[f"{name}_{n}"]) for n in "qkv")
    S0 = _warm_state(float(z[f"{name}_state_scale"][0]))
    y, S = orc.gated_delta_rule(q, k, v, z[f"{name}_g"], z[f"{name}_beta"], S0, np.float64)
    np.testing.assert_allclose(y.sum(axis=2), z[f"{name}_y_sum"], rtol=0, atol=1e-12)
    np.testing.assert_allclose(S.sum(axis=2), z[f"{name}_S_sum"], rtol=0, atol=1e-12)
    np.testing.assert_allclose(y, z[f"{name}_y"], rtol=2e-7, atol=1e-9)
    np.testing.assert_allclose(S[:, ::16, :], z[f"{name}_S_rows"], rtol=2e-7, atol=1e-9)


def test_bf16_round_ties_to_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.0e38, 1e-40], np.float32)
    r = orc.bf16_round(x)
    assert r[0] == 1.0 and r[1] == 1.0 and r[2] == np.float32(1.015625) and r[3] == -2.5
    assert np.all(orc.bf16_from_bits(orc.bf16_bits(r)) == r)


def test_gate_functions_are_bf16_valued_and_monotone():
    x = orc.bf16_round(np.linspace(-20, 20, 4001))
    for f in (orc.sigmoid_bf16, orc.softplus_bf16, orc.silu_bf16):
        y = f(x)
        assert np.all(orc.bf16_round(y) == y)
    s = orc.sigmoid_bf16(x)
    assert np.all(np.diff(s) >= 0) and s[0] >= 0 and s[-1] <= 1
    assert np.allclose(s, 1 / (1 + np.exp(-x.astype(np.float64))), atol=8e-3)
    assert np.allclose(orc.softplus_bf16(x), np.log1p(np.exp(x.astype(np.float64))), rtol=8e-3, atol=4e-3)


def test_chunked_form_equals_sequential_rule_fp64():
    """The chunk-64 WY/UT algebra (gdn_nax.py:3-10) reproduces the sequential rule, including a partial last chunk and a
    non-zero initial state, with decays as extreme as the benchmark's."""
    c = synth.config1(seed=0, T=200)
    lg = orc.log_decay(c["A_log"], c["a"][0], c["dt_bias"])
    beta = orc.beta_gate(c["b"][0])
    S0 = (np.random.default_rng(5).standard_normal((16, 128, 128)) * 0.02)
    y_ref, S_ref = orc.gated_delta_rule(c["q"][0], c["k"][0], c["v"][0], np.exp(lg.astype(np.float64)), beta, S0)
    y, S = orc.chunked_rule(c["q"][0], c["k"][0], c["v"][0], lg, beta, S0, C=64)
    assert orc.max_err_scaled(y, y_ref) < 1e-12
    assert orc.max_err_scaled(S, S_ref) < 1e-12
    assert lg.min() < -20, "the synthetic decays must exercise underflowing in-chunk products"


def test_fp32_rule_close_to_fp64():
    c = synth.config1(seed=0, T=64)
    g = orc.compute_g(c["A_log"], c["a"][0], c["dt_bias"])
    beta = orc.beta_gate(c["b"][0])
    y64, S64 = orc.gated_delta_rule(c["q"][0], c["k"][0], c["v"][0], g, beta, c["state"][0], np.float64)
    y32, S32 = orc.gated_delta_rule(c["q"][0], c["k"][0], c["v"][0], g, beta, c["state"][0], np.float32)
    assert orc.max_err_scaled(y32, y64) < 1e-5 and orc.max_err_scaled(S32, S64) < 1e-5


def test_split_sequence_equals_resume_from_state():
    """Prefix resume == split prefill (tests/prefix_cache.py:85-97 of the reference): running T tokens equals running the first
    T1 and continuing from the carried state."""
    c = synth.config1(seed=3, T=96)
    g = orc.compute_g(c["A_log"], c["a"][0], c["dt_bias"])
    beta = orc.beta_gate(c["b"][0])
    q, k, v = c["q"][0], c["k"][0], c["v"][0]
    y, S = orc.gated_delta_rule(q, k, v, g, beta, c["state"][0])
    y1, S1 = orc.gated_delta_rule(q[:64], k[:64], v[:64], g[:64], beta[:64], c["state"][0])
    y2, S2 = orc.gated_delta_rule(q[64:], k[64:], v[64:], g[64:], beta[64:], S1)
    assert np.array_equal(np.concatenate([y1, y2]), y) and np.array_equal(S2, S)


def test_deltanet_m_tokens_equal_m_single_calls():
    """verify(M) == M x verify(1): snapshots, conv windows and outputs (tests/verify.py of the reference)."""
    c = synth.config2(B=1, seed=1, M=3)
    y, _, cs, st = orc.deltanet(c["proj"], c["conv"][0], c["conv_w"], c["A_log"], c["dt_bias"], c["state"][0])
    win, S = c["conv"][0], c["state"][0]
    for j in range(3):
        y1, _, cs1, st1 = orc.deltanet(c["proj"][j:j + 1], win, c["conv_w"], c["A_log"], c["dt_bias"], S)
        assert np.array_equal(y1[0], y[j]) and np.array_equal(cs1[0], cs[j]) and np.array_equal(st1[0], st[j])
        win, S = cs1[0], st1[0]
    assert np.array_equal(cs[2], c["proj"][:, :6144])          # after 3 tokens the window is exactly the 3 new rows


def test_attention_rows_match_masked_softmax():
    rng = np.random.default_rng(2)
    ctx, M = 37, 3
    q = synth.bf16r(rng.standard_normal((M, 8, 256)))
    kn, vn = synth.bf16r(rng.standard_normal((M, 2, 256))), synth.bf16r(rng.standard_normal((M, 2, 256)))
    kc, vc = synth.bf16r(rng.standard_normal((2, ctx, 256))), synth.bf16r(rng.standard_normal((2, ctx, 256)))
    o = orc.attn_rows(q, kn, vn, kc, vc)
    K = np.concatenate([kc, kn.transpose(1, 0, 2)], axis=1)     # [2, ctx+M, 256]
    V = np.concatenate([vc, vn.transpose(1, 0, 2)], axis=1)
    for j in range(M):
        for h in range(8):
            s = K[h // 4] @ q[j, h].astype(np.float64) / 16.0
            s[ctx + j + 1:] = -np.inf                           # bool mask kv_idx <= pos + row (fast.py:58)
            p = np.exp(s - s.max())
            assert np.allclose(o[j, h], (p / p.sum()) @ V[h // 4], atol=1e-12)


def test_accept_length():
    toks = np.array([[5, 1, 2, 3], [5, 1, 9, 3], [5, 7, 2, 3], [5, 1, 2, 8]])
    ids = np.array([[1, 2, 3, 4], [1, 2, 3, 4], [1, 2, 3, 4], [1, 2, 3, 4]])
    assert orc.accept_length(toks, ids).tolist() == [3, 1, 0, 2]


def test_prefill_attention_oracle_equals_the_decode_oracle_row_by_row():
    """The causal prefill oracle (qwen35/model.py:165) against the decode oracle (qwen35/batch.py:141-227) used one query at a time: query i
    of a chunk that starts at `pos` sees the pos + i cached keys and itself."""
    rng = np.random.default_rng(3)
    S, pos = 9, 5
    q = synth.bf16r(rng.standard_normal((S, 8, 256)))
    K = synth.bf16r(rng.standard_normal((2, pos + S, 256)))
    V = synth.bf16r(rng.standard_normal((2, pos + S, 256)))
    full = orc.prefill_attention(q, K, V, pos)
    for i in range(S):
        n = pos + i
        row = orc.attn_rows(q[i:i + 1], K[:, n][None], V[:, n][None], K[:, :n], V[:, :n])
        assert np.allclose(full[i], row[0], rtol=1e-12, atol=1e-12)


def test_gated_norm_oracle_properties():
    """silu(z) * w * y / rms(y) (qwen35/prefill.py:137-157): scaling y leaves the result unchanged up to the epsilon, a zero gate
    input gives zero, and the result is bf16-valued."""
    rng = np.random.default_rng(4)
    y = synth.bf16r(rng.standard_normal((3, 2048)))
    proj = synth.bf16r(rng.standard_normal((3, 8224)))
    gw = (1.0 + 0.1 * rng.standard_normal(128)).astype(np.float32)
    out = orc.gated_norm(y, proj, gw)
    assert out.shape == (3, 2048) and np.array_equal(out, synth.bf16r(out))
    out2 = orc.gated_norm(synth.bf16r(4.0 * y), proj, gw)            # a power of two: exact in bf16
    assert np.max(np.abs(out2.astype(np.float64) - out)) <= 2.0 ** -7 * np.max(np.abs(out))
    proj0 = proj.copy(); proj0[:, 6144:8192] = 0
    assert not np.any(orc.gated_norm(y, proj0, gw))
