"""The C/OpenMP restatement (the timed CPU baseline) agrees with the numpy oracle."""
import numpy as np

from oracle import build_oracle as co
from oracle import gdn_oracle as orc
from qwen_tailor_b200 import synth


def test_c_decode_step_matches_numpy_oracle():
    B = 3
    c = synth.config2(B=B, seed=1)
    slots = np.array([2, 0, 1], np.int32)
    pos = np.array([4, 7, 0], np.int32)
    conv_pool = np.zeros((B * 2, 3, 6144), np.float32)
    ssm = np.zeros((B, 16, 128, 128), np.float32)
    for b in range(B):
        conv_pool[slots[b] * 2 + (pos[b] & 1)] = c["conv"][b]
        ssm[slots[b]] = c["state"][b]
    cp_bits = orc.bf16_bits(conv_pool)
    y_bits = co.deltanet_b(orc.bf16_bits(c["proj"]), cp_bits, orc.bf16_bits(c["conv_w"]), c["A_log"], c["dt_bias"], ssm, slots, pos)
    for b in range(B):
        y_ref, _, cs_ref, st_ref = orc.deltanet(c["proj"][b:b + 1], c["conv"][b], c["conv_w"], c["A_log"], c["dt_bias"], c["state"][b], np.float32)
        assert orc.max_err_scaled(ssm[slots[b]], st_ref[0]) < 2e-6
        assert orc.rel_l2(orc.bf16_from_bits(y_bits[b]), y_ref[0]) < 2e-3
        assert np.array_equal(orc.bf16_from_bits(cp_bits[slots[b] * 2 + ((pos[b] & 1) ^ 1)]), cs_ref[0])


def test_c_rule_matches_numpy_oracle():
    c = synth.config1(seed=0, T=40)
    g = orc.compute_g(c["A_log"], c["a"], c["dt_bias"])
    beta = orc.beta_gate(c["b"])
    S = c["state"].copy()
    y_bits = co.gated_delta_rule(orc.bf16_bits(c["q"]), orc.bf16_bits(c["k"]), orc.bf16_bits(c["v"]), g, beta, S)
    y_ref, S_ref = orc.gated_delta_rule(c["q"][0], c["k"][0], c["v"][0], g[0], beta[0], c["state"][0], np.float64)
    assert orc.max_err_scaled(S[0], S_ref) < 1e-5
    assert orc.rel_l2(orc.bf16_from_bits(y_bits[0]), y_ref) < 2e-3


def test_c_attention_row_matches_numpy_oracle():
    rng = np.random.default_rng(0)
    n = 300
    q = synth.bf16r(rng.standard_normal((8, 256)))
    K, V = synth.bf16r(rng.standard_normal((2, n, 256))), synth.bf16r(rng.standard_normal((2, n, 256)))
    o = orc.bf16_from_bits(co.attn_row(orc.bf16_bits(q), orc.bf16_bits(K), orc.bf16_bits(V)))
    ref = orc.attn_rows(q[None], K[:, -1:].transpose(1, 0, 2), V[:, -1:].transpose(1, 0, 2), K[:, :-1], V[:, :-1])[0]
    assert orc.rel_l2(o, ref) < 2e-3
