"""GPU parity of the elementwise glue kernels (attention qkv prep / output gate, prefill conv prep, gated RMSNorm) and of a
whole GDN prefill layer assembled from them (conv_prep -> gates -> chunked rule -> gated norm) against the oracle."""
import numpy as np
import pytest
import torch

from conftest import bf16_dev, f32_dev, host, i32_dev
from oracle import gdn_oracle as orc
from qwen_tailor_b200 import synth
from qwen_tailor_b200.attn_glue import gate_out, qkv_prep
from qwen_tailor_b200.gdn_nax import gdn_chunked
from qwen_tailor_b200.kernels import deltanet
from qwen_tailor_b200.prefill import conv_prep, gated_norm

pytestmark = pytest.mark.gpu


def _close_bf16(got, ref, frac=0.02):
    """bf16 results of the same chain of bf16-rounded ops: identical except on a small fraction of the elements, where an fp32
    library function (exp, sqrt) differed in the last place before a rounding; such a flip is one bf16 step, two when it is
    carried through a second rounding or sits on a power of two."""
    assert orc.bf16_ulp_distance(got, ref).max() <= 2.0 + 1e-6
    assert (got != ref).mean() < frac


def test_qkv_prep_matches_oracle(dev):
    rng = np.random.default_rng(0)
    R = 9
    qkv = synth.bf16r(rng.standard_normal((R, 5120)))
    qn = (1.0 + 0.1 * rng.standard_normal(256)).astype(np.float32)
    kn = (1.0 + 0.1 * rng.standard_normal(256)).astype(np.float32)
    pos = np.array([0, 1, 2, 31, 32, 300, 1023, 4095, 8191], np.int32)
    q, gate, k, v = qkv_prep(bf16_dev(qkv, dev), f32_dev(qn, dev), f32_dev(kn, dev), i32_dev(pos, dev))
    qr, gr, kr, vr = orc.qkv_prep(qkv, qn, kn, pos)
    assert np.array_equal(host(gate), gr) and np.array_equal(host(v), vr)
    _close_bf16(host(q)[..., 64:], qr[..., 64:])                   # dims that are only normed
    _close_bf16(host(k)[..., 64:], kr[..., 64:])
    # rotated dims.  The kernel forms the angle pos * theta^(-i/32) in fp32 like the reference's rope op, the oracle in fp64: the
    # product carries a relative error of 2^-23 (exp2 and one multiply), i.e. up to pos * 2^-23 radians, which moves a rotated
    # pair of radius r by that much times r; on top of it one bf16 rounding step (2^-8 of the value) where the two disagree.
    for got, ref in ((host(q), qr), (host(k), kr)):
        radius = np.sqrt(ref[..., :32].astype(np.float64) ** 2 + ref[..., 32:64].astype(np.float64) ** 2)
        radius = np.concatenate([radius, radius], axis=-1) * (1 + 2.0 ** -7)
        bound = pos.astype(np.float64)[:, None, None] * 2.0 ** -22 * radius + 2.0 ** -7 * np.abs(ref[..., :64]) + 1e-30
        assert np.all(np.abs(got[..., :64].astype(np.float64) - ref[..., :64]) <= bound)
    small = pos < 64
    _close_bf16(host(q)[small][..., :64], qr[small][..., :64], frac=0.05)
    _close_bf16(host(k)[small], kr[small], frac=0.05)


def test_gate_out_matches_oracle(dev):
    rng = np.random.default_rng(1)
    o = synth.bf16r(rng.standard_normal((7, 2048)))
    g = synth.bf16r(rng.standard_normal((7, 2048)) * 3)
    _close_bf16(host(gate_out(bf16_dev(o, dev), bf16_dev(g, dev))), orc.gate_out(o, g), frac=0.01)


@pytest.mark.parametrize("S", [1, 2, 3, 5, 64, 200])
def test_conv_prep_matches_oracle_and_decode_kernel(dev, S):
    """conv_prep == the oracle, and row for row == what the decode kernel computes for the same tokens (its conv window after S
    tokens equals conv_prep's new window): the reference's "fused == unfused" contract (tests/gdn_fuse.py)."""
    rng = np.random.default_rng(S)
    c = synth.config2(B=1, seed=S, M=1)
    proj = synth.bf16r(rng.standard_normal((S, 8224)))
    q, k, v, new = conv_prep(bf16_dev(proj, dev), bf16_dev(c["conv"], dev), bf16_dev(c["conv_w"], dev))
    qr, kr, vr, newr = orc.conv_prep(proj, c["conv"][0], c["conv_w"])
    assert np.array_equal(host(new), newr)
    _close_bf16(host(q), qr)
    _close_bf16(host(k), kr)
    _close_bf16(host(v), vr, frac=0.005)
    if S <= 5:
        _, cs, _ = deltanet(bf16_dev(proj, dev), bf16_dev(c["conv"], dev), bf16_dev(c["conv_w"], dev), f32_dev(c["A_log"], dev), f32_dev(c["dt_bias"], dev),
                            f32_dev(c["state"], dev), i32_dev([0], dev))
        assert torch.equal(cs[S - 1], new)


def test_gated_norm_matches_oracle(dev):
    rng = np.random.default_rng(2)
    S = 33
    y = synth.bf16r(rng.standard_normal((S, 2048)) * 0.05)
    proj = synth.bf16r(rng.standard_normal((S, 8224)))
    gw = (1.0 + 0.2 * rng.standard_normal(128)).astype(np.float32)
    out = gated_norm(bf16_dev(y, dev), bf16_dev(proj, dev), f32_dev(gw, dev))
    _close_bf16(host(out), orc.gated_norm(y, proj, gw), frac=0.01)


def test_prefill_layer_pipeline(dev):
    """A whole GDN prefill layer: proj -> conv_prep -> gdn_chunked (gates from proj) -> gated_norm, against the oracle chain, and
    the state / window it leaves equal to what token-by-token decoding of the same rows leaves (within the state tolerance)."""
    rng = np.random.default_rng(3)
    S = 130
    c = synth.config2(B=1, seed=3, M=1)
    proj = synth.bf16r(rng.standard_normal((S, 8224)))
    gw = np.ones(128, np.float32)
    pj, cw = bf16_dev(proj, dev), bf16_dev(c["conv_w"], dev)
    A_log, dtb = f32_dev(c["A_log"], dev), f32_dev(c["dt_bias"], dev)
    q, k, v, new = conv_prep(pj, bf16_dev(c["conv"], dev), cw)
    y, st = gdn_chunked(q, k, v, pj, A_log, dtb, f32_dev(c["state"], dev))
    out = gated_norm(y, pj, f32_dev(gw, dev))
    qr, kr, vr, _ = orc.conv_prep(proj, c["conv"][0], c["conv_w"])
    g = orc.compute_g(c["A_log"], proj[:, 8208:8224], c["dt_bias"])
    beta = orc.beta_gate(proj[:, 8192:8208])
    y_ref, s_ref = orc.gated_delta_rule(qr, kr, vr, g, beta, c["state"][0], np.float64)
    assert orc.max_err_scaled(host(st[0]), s_ref) < 1e-4
    assert orc.rel_l2(host(y), y_ref) < 2.5e-3
    out_ref = orc.gated_norm(orc.bf16_round(y_ref.reshape(S, 2048).astype(np.float32)), proj, gw)
    assert orc.rel_l2(host(out), out_ref) < 4e-3
    # decode the same tokens one by one from the same start: final state and window agree with the prefill
    cs, ss = bf16_dev(c["conv"], dev), f32_dev(c["state"], dev)
    sel = i32_dev([0], dev)
    for t in range(0, S, 4):
        _, cs4, ss4 = deltanet(pj[t:t + 4], cs, cw, A_log, dtb, ss, sel)
        cs, ss = cs4[-1:].contiguous(), ss4[-1:].contiguous()
    assert torch.equal(cs[0], new)
    assert orc.max_err_scaled(host(ss[0]), host(st[0])) < 1e-4
