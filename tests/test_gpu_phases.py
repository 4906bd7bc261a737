"""GPU tests of the two-phase prefill API (prep_a / phase_a / phase_b of qwen35/gdn_nax.py): the reference's bit contract
"prep_a == conv_prep followed by phase A" for its partial-chunk lengths (tests/gdn_fuse.py:29-40), phase_b on those outputs ==
gdn_chunked, and every one of the 18 per-layer seeds of benchmark configuration 3 against the oracle."""
import numpy as np
import pytest
import torch

from conftest import bf16_dev, f32_dev, host, i32_dev
from oracle import gdn_oracle as orc
from qwen_tailor_b200 import _lib, synth
from qwen_tailor_b200.gated_delta import gates
from qwen_tailor_b200.gdn_nax import REC_BYTES, gdn_chunked, gdn_chunked_varlen, phase_a, phase_a_varlen, phase_b, phase_b_varlen, prep_a
from qwen_tailor_b200.prefill import conv_prep

pytestmark = pytest.mark.gpu


def _layer_inputs(dev, S, seed):
    rng = np.random.default_rng(seed)
    c = synth.config2(B=1, seed=seed, M=1)
    proj = synth.bf16r(rng.standard_normal((S, 8224)))
    st0 = (rng.standard_normal((1, 16, 128, 128)) * 0.02).astype(np.float32)
    return (bf16_dev(proj, dev), bf16_dev(c["conv"][0], dev), bf16_dev(c["conv_w"], dev), f32_dev(c["A_log"], dev), f32_dev(c["dt_bias"], dev),
            f32_dev(st0, dev))


@pytest.mark.parametrize("S", [2048, 2000, 37, 16, 5])
def test_prep_a_is_bit_identical_to_conv_prep_then_phase_a(dev, S):
    """tests/gdn_fuse.py:29-40 of the reference: the fused kernel's q, k, v and phase-A outputs equal the unfused path bit for bit,
    and phase_b on them equals gdn_chunked."""
    proj, conv, cw, A_log, dtb, st0 = _layer_inputs(dev, S, seed=S)
    q, k, v, Tb, Am, gv = prep_a(proj, conv, cw.reshape(6144, 1, 4), A_log, dtb)
    q2, k2, v2, _ = conv_prep(proj, conv, cw)
    assert torch.equal(q, q2) and torch.equal(k, k2) and torch.equal(v, v2)
    Tb2, Am2, gv2 = phase_a(q2, k2, proj, A_log, dtb)
    nvalid = (S + 63) // 64 * 16 * REC_BYTES                       # the records of the sequence's chunks (the buffer has one spare slot)
    assert Tb.dtype == torch.uint8 and Tb.numel() >= nvalid and torch.equal(Tb[:nvalid], Tb2[:nvalid])
    assert torch.equal(gv, gv2) and Am.numel() == 0
    y, st = phase_b(q, k, v, Tb, Am, gv, st0)
    y2, st2 = gdn_chunked(q2, k2, v2, proj, A_log, dtb, st0)
    assert y.shape == (S, 16, 128) and st.shape == (1, 16, 128, 128)
    assert torch.equal(y, y2) and torch.equal(st, st2)
    assert _lib.device_status() == 0


def test_prep_a_phase_b_match_the_oracle(dev):
    """The reference's default prefill path (qwen35/prefill.py:251-253) end to end against the fp64 oracle."""
    S = 300
    rng = np.random.default_rng(11)
    c = synth.config2(B=1, seed=11, M=1)
    proj = synth.bf16r(rng.standard_normal((S, 8224)))
    st0 = (rng.standard_normal((16, 128, 128)) * 0.02).astype(np.float32)
    q, k, v, Tb, Am, gv = prep_a(bf16_dev(proj, dev), bf16_dev(c["conv"][0], dev), bf16_dev(c["conv_w"], dev), f32_dev(c["A_log"], dev),
                                 f32_dev(c["dt_bias"], dev))
    y, st = phase_b(q, k, v, Tb, Am, gv, f32_dev(st0[None], dev))
    qr, kr, vr, _ = orc.conv_prep(proj, c["conv"][0], c["conv_w"])
    g = orc.compute_g(c["A_log"], proj[:, 8208:8224], c["dt_bias"])
    beta = orc.beta_gate(proj[:, 8192:8208])
    y_ref, s_ref = orc.gated_delta_rule(qr, kr, vr, g, beta, st0, np.float64)
    assert orc.max_err_scaled(host(st[0]), s_ref) < 1e-4
    assert orc.rel_l2(host(y), y_ref) < 2.5e-3                     # q, k, v themselves differ from the oracle's by bf16 rounding flips


def test_phase_a_records_hold_the_inverse(dev):
    """Phase A against numpy: Tb = (I + L)^-1 diag(beta) from the hi + lo halves of a record, and the gate vectors."""
    T = 150
    c = synth.config1(seed=21, T=T)
    k = bf16_dev(c["k"][0], dev)
    _, lg, beta = gates(bf16_dev(c["a"][0], dev), bf16_dev(c["b"][0], dev), f32_dev(c["A_log"], dev), f32_dev(c["dt_bias"], dev))
    rec = host(phase_a_varlen(k, lg, beta, i32_dev([0, T], dev))).astype(np.uint8)
    lgn, betan = host(lg).astype(np.float64), host(beta).astype(np.float64)
    for chunk, head in ((0, 0), (1, 7), (2, 15)):                    # chunk 2 is partial (22 tokens)
        r = rec[(chunk * 16 + head) * REC_BYTES:(chunk * 16 + head + 1) * REC_BYTES]
        t0, n = chunk * 64, min(64, T - chunk * 64)
        K = c["k"][0][t0:t0 + n, head].astype(np.float64)
        Lc = np.cumsum(lgn[t0:t0 + n, head])
        b = betan[t0:t0 + n, head]
        L = np.tril(b[:, None] * np.exp(Lc[:, None] - Lc[None, :]) * (K @ K.T), -1)
        want = np.linalg.inv(np.eye(n) + L) * b[None, :]

        def image(buf):                                            # [64][64] bf16 operand image with the 128-byte swizzle
            raw = np.frombuffer(buf.tobytes(), np.uint16).reshape(64, 8, 8)      # row, 16-byte piece, element
            out = np.empty((64, 64), np.float32)
            for i in range(64):
                for p in range(8):
                    out[i, ((p ^ (i & 7)) * 8):((p ^ (i & 7)) * 8 + 8)] = (raw[i, p].astype(np.uint32) << 16).view(np.float32)
            return out.astype(np.float64)
        got = image(r[:8192]) + image(r[8192:16384])
        assert np.abs(got[:n, :n] - want).max() < 2e-5 * max(1.0, np.abs(want).max())
        assert np.all(got[n:] == 0) and np.all(got[:, n:] == 0)
        gvec = np.frombuffer(r[16384:].tobytes(), np.float32).reshape(3, 64)
        assert np.allclose(gvec[0, :n], Lc * np.log2(np.e), rtol=1e-5, atol=1e-5)
        assert np.allclose(gvec[1, :n], np.exp(Lc), rtol=1e-4, atol=1e-30)
        assert np.allclose(gvec[2, :n], np.exp(Lc[-1] - Lc), rtol=1e-4, atol=1e-30)


def test_phase_split_equals_the_combined_call_on_a_packed_batch(dev):
    lens = [70, 0, 64, 1, 129]
    rng = np.random.default_rng(5)
    A_log, dt_bias = synth.layer_params(rng)
    qn, kn, vn, an, bn = synth.gdn_tokens(rng, sum(lens))
    cu = i32_dev(np.concatenate([[0], np.cumsum(lens)]), dev)
    q, k, v = (bf16_dev(x, dev) for x in (qn, kn, vn))
    _, lg, beta = gates(bf16_dev(an, dev), bf16_dev(bn, dev), f32_dev(A_log, dev), f32_dev(dt_bias, dev))
    rec = phase_a_varlen(k, lg, beta, cu)
    y, s = phase_b_varlen(q, k, v, rec, cu)
    y2, s2 = gdn_chunked_varlen(q, k, v, lg, beta, cu)
    assert torch.equal(y, y2) and torch.equal(s, s2)
    with pytest.raises(ValueError):                                  # a record buffer that is too small is refused before any launch
        phase_b_varlen(q, k, v, rec[:100], cu)
    assert _lib.device_status() == 0


@pytest.mark.parametrize("layer", list(range(18)))
def test_config3_every_layer_seed(dev, layer):
    """Benchmark configuration 3, T = 2048, per-layer seeds 100..117.  Layer 0 (seed 100) is checked on all 16 heads in
    test_gpu_prefill.py; here every layer is checked against the fp64 oracle on four of its heads (the sequential oracle takes a
    few seconds per head at this length), and on finiteness of everything."""
    T = 2048
    c = synth.config3_layer(layer, T)
    q, k, v = (bf16_dev(c[n], dev) for n in ("q", "k", "v"))
    _, lg, beta = gates(bf16_dev(c["a"], dev), bf16_dev(c["b"], dev), f32_dev(c["A_log"], dev), f32_dev(c["dt_bias"], dev))
    y, s = gdn_chunked_varlen(q, k, v, lg, beta, i32_dev([0, T], dev))
    assert bool(torch.isfinite(s).all()) and bool(torch.isfinite(y.float()).all())
    heads = [(layer + 4 * i) % 16 for i in range(4)]
    g = orc.compute_g(c["A_log"], c["a"], c["dt_bias"])[:, heads]
    bt = orc.beta_gate(c["b"])[:, heads]
    y_ref, s_ref = orc.gated_delta_rule(c["q"][:, heads], c["k"][:, heads], c["v"][:, heads], g, bt, np.zeros((4, 128, 128)), np.float64)
    assert orc.max_err_scaled(host(s[0])[heads], s_ref) < 1e-4
    assert orc.rel_l2(host(y)[:, heads], y_ref) < 2e-3
    assert _lib.device_status() == 0


@pytest.mark.parametrize("S", [2048, 2000, 37, 5])
def test_gated_norm_fused_into_phase_b_equals_the_separate_kernel(dev, S):
    """The reference's layer ends with ``gated_norm(out, proj, gnorm)`` on the output of phase_b (qwen35/prefill.py:253-264).  With the
    norm applied in phase B's y store the result has the same bits as the two calls, and the state is untouched by the option."""
    from qwen_tailor_b200.prefill import gated_norm
    proj, conv, cw, A_log, dtb, st0 = _layer_inputs(dev, S, seed=100 + S)
    gw = f32_dev(1.0 + 0.1 * np.random.default_rng(S).standard_normal(128).astype(np.float32), dev)
    q, k, v, Tb, Am, gv = prep_a(proj, conv, cw.reshape(6144, 1, 4), A_log, dtb)
    y, st = phase_b(q, k, v, Tb, Am, gv, st0)
    want = gated_norm(y, proj, gw)
    got, st2 = phase_b(q, k, v, Tb, Am, gv, st0, gate_proj=proj, gate_w=gw)
    assert torch.equal(got.reshape(S, 2048), want) and torch.equal(st, st2)
    assert _lib.device_status() == 0


def test_gated_norm_fused_on_a_packed_batch_and_head_range(dev):
    """Packed ragged sequences, a head sub-range: the fused store only touches the rows and heads that the call owns."""
    from qwen_tailor_b200.prefill import gated_norm
    lens = [130, 64, 1, 77]
    T = sum(lens)
    rng = np.random.default_rng(7)
    proj = bf16_dev(synth.bf16r(rng.standard_normal((T, 8224))), dev)
    gw = f32_dev(1.0 + 0.1 * rng.standard_normal(128).astype(np.float32), dev)
    q = bf16_dev(synth.bf16r(rng.standard_normal((T, 16, 128)) * 0.088), dev)
    k = bf16_dev(synth.bf16r(rng.standard_normal((T, 16, 128)) * 0.088), dev)
    v = bf16_dev(synth.bf16r(rng.standard_normal((T, 16, 128))), dev)
    lg = f32_dev(-np.abs(rng.standard_normal((T, 16))).astype(np.float32) * 0.05, dev)
    beta = f32_dev(rng.uniform(0.1, 0.9, (T, 16)).astype(np.float32), dev)
    cu = i32_dev(np.concatenate([[0], np.cumsum(lens)]).astype(np.int32), dev)
    y, st = gdn_chunked_varlen(q, k, v, lg, beta, cu)
    want = gated_norm(y, proj, gw).reshape(T, 16, 128)
    got = torch.full_like(y, 3.0)
    _, st2 = gdn_chunked_varlen(q, k, v, lg, beta, cu, head_lo=4, head_hi=12, y=got, gate_proj=proj, gate_w=gw)
    assert torch.equal(got[:, 4:12], want[:, 4:12])
    assert torch.all(got[:, :4] == 3.0) and torch.all(got[:, 12:] == 3.0)
    assert torch.equal(st2[:, 4:12], st[:, 4:12])
