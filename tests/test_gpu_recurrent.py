"""GPU parity of the ops-level API (compute_g, normalize_qk, gated_delta_update) against the oracle and the reference's
rec64 known-answer vectors; shape list and error behaviour of the reference's tests/gated_delta.py."""
from pathlib import Path

import numpy as np
import pytest
import torch

from conftest import bf16_dev, f32_dev, host
from oracle import gdn_oracle as orc
from qwen_tailor_b200 import synth
from qwen_tailor_b200.gated_delta import compute_g, gated_delta_update, gates, normalize_qk
from test_oracle import GOLD, _warm_state

pytestmark = pytest.mark.gpu


def test_gates_bit_exact_over_all_bf16_inputs(dev):
    """beta and the bf16 part of the decay gate are evaluated op by op in bf16: compare every finite bf16 input in (-60, 60)
    with the oracle.  The fp32 exp/log1p of two libraries may differ in the last place before rounding, so a handful of inputs
    may land on the other side of a bf16 rounding boundary."""
    bits = (np.arange(65536, dtype=np.uint32) << 16).view(np.float32)
    x = bits[np.isfinite(bits) & (np.abs(bits) < 60)]
    n = (len(x) // 16) * 16
    x = x[:n].reshape(-1, 16)
    A_log = np.zeros(16, np.float32)
    dtb = np.zeros(16, np.float32)
    g, lg, beta = gates(bf16_dev(x, dev), bf16_dev(x, dev), f32_dev(A_log, dev), f32_dev(dtb, dev))
    beta_ref = orc.beta_gate(x)
    lg_ref = orc.log_decay(A_log, x, dtb)
    assert (host(beta) != beta_ref).mean() < 2e-3 and np.abs(host(beta) - beta_ref).max() <= 2 ** -8
    assert (host(lg) != lg_ref).mean() < 2e-3 and np.allclose(host(lg), lg_ref, rtol=8e-3, atol=1e-6)
    assert np.allclose(host(g), np.exp(host(lg).astype(np.float64)), rtol=1e-6, atol=1e-30)


def test_normalize_qk(dev):
    rng = np.random.default_rng(0)
    q = synth.bf16r(rng.standard_normal((2, 5, 16, 128)) * 2)
    k = synth.bf16r(rng.standard_normal((2, 5, 16, 128)) * 2)
    qn, kn = normalize_qk(bf16_dev(q, dev), bf16_dev(k, dev), inv_scale=128 ** -0.5, eps=1e-6)
    qr, kr = orc.normalize_qk(q, k)
    assert orc.bf16_ulp_distance(host(qn), qr).max() <= 1 and (host(qn) != qr).mean() < 0.02
    assert orc.bf16_ulp_distance(host(kn), kr).max() <= 1 and (host(kn) != kr).mean() < 0.02
    with pytest.raises(ValueError):
        normalize_qk(bf16_dev(q[..., :64], dev), bf16_dev(k[..., :64], dev), inv_scale=0.1, eps=1e-6)


@pytest.mark.parametrize("B,T", [(1, 1), (1, 3), (2, 5), (4, 1), (1, 257), (1, 2048)])
def test_gated_delta_update_shapes(dev, B, T):
    """Shape list of the reference's tests/gated_delta.py:44; random state x 0.1 and state=None."""
    rng = np.random.default_rng(B * 1000 + T)
    A_log, dt_bias = synth.layer_params(rng)
    q, k, v, a, b = synth.gdn_tokens(rng, T, lead=(B,))
    st = (rng.standard_normal((B, 16, 128, 128)) * 0.1).astype(np.float32)
    args = [bf16_dev(x, dev) for x in (q, k, v, a, b)] + [f32_dev(A_log, dev), f32_dev(dt_bias, dev)]
    for state in (st, None):
        y, s = gated_delta_update(*args, None if state is None else f32_dev(state, dev))
        assert y.shape == (B, T, 16, 128) and y.dtype == torch.bfloat16 and s.shape == (B, 16, 128, 128) and s.dtype == torch.float32
        y_ref, y_un, s_ref = orc.gated_delta_update(q, k, v, a, b, A_log, dt_bias, state, np.float64)
        assert orc.max_err_scaled(host(s), s_ref) < 1e-4
        assert orc.rel_l2(host(y), y_un) < 2e-3
        assert orc.max_err_scaled(host(y), y_ref) < 4e-3


def test_config1_parity(dev):
    """Benchmark configuration 1: B=1, T=256, zero state, seed 0."""
    c = synth.config1()
    y, s = gated_delta_update(*[bf16_dev(c[n], dev) for n in ("q", "k", "v", "a", "b")], f32_dev(c["A_log"], dev), f32_dev(c["dt_bias"], dev),
                              f32_dev(c["state"], dev))
    y_ref, y_un, s_ref = orc.gated_delta_update(c["q"], c["k"], c["v"], c["a"], c["b"], c["A_log"], c["dt_bias"], c["state"], np.float64)
    assert orc.max_err_scaled(host(s), s_ref) < 1e-4
    assert orc.rel_l2(host(y), y_un) < 2e-3
    # almost every output equals the correctly rounded fp64 result; the rest sit on the other side of a bf16 rounding boundary
    # (one bf16 step = 2^-8 relative to the element, hence the 4e-3 bound on the scale-normalised maximum)
    exact = (host(y) == y_ref).mean()
    assert exact > 0.99 and orc.max_err_scaled(host(y), y_ref) < 4e-3, exact


@pytest.mark.parametrize("name", ["zero_state", "warm_state"])
def test_rec64_known_answers(dev, name):
    """The CUDA recurrence against the outputs of the reference's own rec64 (tests/golden/rec64_kat.npz)."""
    from qwen_tailor_b200 import _lib
    from qwen_tailor_b200._lib import check, ptr, stream_ptr
    z = np.load(GOLD)
    q, k, v = (orc.bf16_from_bits(z[f"{name}_{n}"]) for n in "qkv")
    T = q.shape[0]
    S0 = _warm_state(float(z[f"{name}_state_scale"][0]))
    qd, kd, vd = (bf16_dev(x[None], dev) for x in (q, k, v))
    g, beta, s0 = f32_dev(z[f"{name}_g"], dev), f32_dev(z[f"{name}_beta"], dev), f32_dev(S0[None], dev)
    y = torch.empty((1, T, 16, 128), dtype=torch.bfloat16, device=dev)
    s = torch.empty((1, 16, 128, 128), dtype=torch.float32, device=dev)
    check(_lib.load().gdn_recurrent(ptr(qd), ptr(kd), ptr(vd), ptr(g), ptr(beta), ptr(s0), ptr(y), ptr(s), 1, T, 16, 16, 128, 128, stream_ptr(dev)), "gdn_recurrent")
    assert orc.rel_l2(host(y[0]), z[f"{name}_y"]) < 2e-3
    assert orc.max_err_scaled(host(s[0])[:, ::16, :], z[f"{name}_S_rows"]) < 1e-4
    assert np.allclose(host(s[0]).astype(np.float64).sum(axis=2), z[f"{name}_S_sum"], atol=2e-4)


def test_unsupported_head_dim_raises(dev):
    rng = np.random.default_rng(0)
    q, k, v, a, b = synth.gdn_tokens(rng, 2, lead=(1,))
    A_log, dt_bias = synth.layer_params(rng)
    with pytest.raises(ValueError):
        gated_delta_update(bf16_dev(q[..., :64], dev), bf16_dev(k[..., :64], dev), bf16_dev(v[..., :64], dev), bf16_dev(a, dev), bf16_dev(b, dev),
                           f32_dev(A_log, dev), f32_dev(dt_bias, dev))
    with pytest.raises(ValueError):
        gated_delta_update(bf16_dev(q, dev), bf16_dev(k, dev), bf16_dev(v, dev), bf16_dev(a, dev), bf16_dev(b, dev), f32_dev(A_log, dev),
                           f32_dev(dt_bias, dev), torch.zeros((1, 16, 128, 128), dtype=torch.bfloat16, device=dev))


def test_cpu_tensors_are_refused():
    with pytest.raises(RuntimeError):
        compute_g(torch.zeros(16), torch.zeros((1, 1, 16), dtype=torch.bfloat16), torch.zeros(16))
