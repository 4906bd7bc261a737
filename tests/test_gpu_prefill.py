"""GPU parity of the chunked (tcgen05) prefill kernel: against the fp64 oracle, against the sequential CUDA kernel, and the
reference's bit contracts (partial-chunk lengths of tests/gdn_fuse.py:29-40; resume == split prefill of tests/prefix_cache.py)."""
import numpy as np
import pytest
import torch

from conftest import bf16_dev, f32_dev, host, i32_dev
from oracle import gdn_oracle as orc
from qwen_tailor_b200 import _lib, synth
from qwen_tailor_b200.gated_delta import gated_delta_update, gates
from qwen_tailor_b200.gdn_nax import gdn_chunked, gdn_chunked_varlen

pytestmark = pytest.mark.gpu

Y_REL_L2, Y_MAX, STATE_TOL = 2e-3, 4e-3, 1e-4


def _dev_case(dev, c, lead=False):
    sl = (lambda x: x[0]) if lead else (lambda x: x)
    q, k, v, a, b = (bf16_dev(sl(c[n]), dev) for n in ("q", "k", "v", "a", "b"))
    A_log, dt_bias = f32_dev(c["A_log"], dev), f32_dev(c["dt_bias"], dev)
    _, lg, beta = gates(a, b, A_log, dt_bias)
    return q, k, v, lg, beta


def _oracle(c, T0=0, T1=None, S0=None):
    q, k, v, a, b = (c[n][0] if c[n].ndim == 4 or (n in "ab" and c[n].ndim == 3) else c[n] for n in ("q", "k", "v", "a", "b"))
    g = orc.compute_g(c["A_log"], a, c["dt_bias"])
    beta = orc.beta_gate(b)
    S0 = np.zeros((16, 128, 128)) if S0 is None else S0
    return orc.gated_delta_rule(q[T0:T1], k[T0:T1], v[T0:T1], g[T0:T1], beta[T0:T1], S0, np.float64)


@pytest.mark.parametrize("T", [256, 64, 1, 5, 16, 37, 63, 65, 128, 200])
def test_chunked_matches_oracle(dev, T):
    """Configuration 1 (T = 256) and the partial-chunk lengths: zero initial state, seed 0."""
    c = synth.config1(seed=0, T=T)
    q, k, v, lg, beta = _dev_case(dev, c, lead=True)
    y, s = gdn_chunked_varlen(q, k, v, lg, beta, i32_dev([0, T], dev))
    y_ref, s_ref = _oracle(c)
    assert y.shape == (T, 16, 128) and s.shape == (1, 16, 128, 128)
    assert orc.max_err_scaled(host(s[0]), s_ref) < STATE_TOL
    assert orc.rel_l2(host(y), y_ref) < Y_REL_L2
    assert orc.max_err_scaled(host(y), orc.bf16_round(y_ref)) < Y_MAX
    assert _lib.device_status() == 0


@pytest.mark.parametrize("T", [2048, 2000])
def test_chunked_long_sequence(dev, T):
    """Configuration 3 sizes (one layer, seed 100): oracle parity and agreement with the sequential CUDA kernel."""
    c = synth.config3_layer(0, T)
    q, k, v, lg, beta = _dev_case(dev, c)
    y, s = gdn_chunked_varlen(q, k, v, lg, beta, i32_dev([0, T], dev))
    y_ref, s_ref = _oracle(c)
    assert orc.max_err_scaled(host(s[0]), s_ref) < STATE_TOL
    assert orc.rel_l2(host(y), y_ref) < Y_REL_L2
    assert orc.max_err_scaled(host(y), orc.bf16_round(y_ref)) < Y_MAX
    y2, s2 = gated_delta_update(q[None], k[None], v[None], bf16_dev(c["a"][None], dev), bf16_dev(c["b"][None], dev), f32_dev(c["A_log"], dev),
                                f32_dev(c["dt_bias"], dev))
    assert orc.max_err_scaled(host(s[0]), host(s2[0])) < STATE_TOL
    assert (host(y) == host(y2[0])).mean() > 0.98


def test_resume_from_state_is_bit_identical_to_unsplit(dev):
    """A prefill resumed from the state after a chunk-aligned prefix equals the unsplit prefill bit for bit (the inter-chunk
    state is the only carried quantity), and a non-zero initial state matches the oracle."""
    T, P = 300, 128
    c = synth.config1(seed=3, T=T)
    q, k, v, lg, beta = _dev_case(dev, c, lead=True)
    y, s = gdn_chunked_varlen(q, k, v, lg, beta, i32_dev([0, T], dev))
    y1, s1 = gdn_chunked_varlen(q[:P].contiguous(), k[:P].contiguous(), v[:P].contiguous(), lg[:P].contiguous(), beta[:P].contiguous(), i32_dev([0, P], dev))
    y2, s2 = gdn_chunked_varlen(q[P:].contiguous(), k[P:].contiguous(), v[P:].contiguous(), lg[P:].contiguous(), beta[P:].contiguous(),
                                i32_dev([0, T - P], dev), init_state=s1)
    assert torch.equal(torch.cat([y1, y2]), y) and torch.equal(s2, s)
    s1_before = s1.clone()
    y_ref, s_ref = _oracle(c, P, T, host(s1[0]).astype(np.float64))
    assert orc.max_err_scaled(host(s2[0]), s_ref) < STATE_TOL and orc.rel_l2(host(y2), y_ref) < Y_REL_L2
    assert torch.equal(s1, s1_before), "the cached state a resume starts from must not be modified"


def test_packed_varlen_equals_individual_runs(dev):
    """Sequences packed by cu_seqlens (including an empty one and partial chunks) give exactly the per-sequence results; resuming
    sequences pick their cached state through init_idx; nothing leaks across sequence boundaries."""
    lens = [70, 0, 64, 1, 129, 33]
    rng = np.random.default_rng(5)
    A_log, dt_bias = synth.layer_params(rng)
    total = sum(lens)
    qn, kn, vn, an, bn = synth.gdn_tokens(rng, total)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    q, k, v = (bf16_dev(x, dev) for x in (qn, kn, vn))
    _, lg, beta = gates(bf16_dev(an, dev), bf16_dev(bn, dev), f32_dev(A_log, dev), f32_dev(dt_bias, dev))
    cache = f32_dev((rng.standard_normal((2, 16, 128, 128)) * 0.02), dev)
    idx = np.array([-1, 1, 0, -1, 1, -1], np.int32)
    y, s = gdn_chunked_varlen(q, k, v, lg, beta, i32_dev(cu, dev), init_state=cache, init_idx=i32_dev(idx, dev))
    for i, n in enumerate(lens):
        a0, a1 = int(cu[i]), int(cu[i + 1])
        init = None if idx[i] < 0 else cache[idx[i]:idx[i] + 1].contiguous()
        if n == 0:
            want = torch.zeros_like(s[i]) if init is None else init[0]
            assert torch.equal(s[i], want)
            continue
        yi, si = gdn_chunked_varlen(q[a0:a1].contiguous(), k[a0:a1].contiguous(), v[a0:a1].contiguous(), lg[a0:a1].contiguous(),
                                    beta[a0:a1].contiguous(), i32_dev([0, n], dev), init_state=init)
        assert torch.equal(y[a0:a1], yi) and torch.equal(s[i], si[0])
    assert _lib.device_status() == 0


def test_head_range_only_touches_its_heads(dev):
    """Head-group sharding: computing heads [4, 8) writes exactly those heads of y / final_state and equals the full run there."""
    T = 100
    c = synth.config1(seed=9, T=T)
    q, k, v, lg, beta = _dev_case(dev, c, lead=True)
    cu = i32_dev([0, T], dev)
    y, s = gdn_chunked_varlen(q, k, v, lg, beta, cu)
    y_part = torch.full_like(y, 7.0)
    s_part = torch.full_like(s, 7.0)
    gdn_chunked_varlen(q, k, v, lg, beta, cu, head_lo=4, head_hi=8, y=y_part, final_state=s_part)
    assert torch.equal(y_part[:, 4:8], y[:, 4:8]) and torch.equal(s_part[:, 4:8], s[:, 4:8])
    assert bool((y_part[:, :4] == 7).all()) and bool((y_part[:, 8:] == 7).all()) and bool((s_part[:, :4] == 7).all()) and bool((s_part[:, 8:] == 7).all())


def test_gdn_chunked_reference_signature(dev):
    """gdn_chunked(q, k, v, proj, A_log, dt_bias, state) with the gates taken from proj columns 8192:8224."""
    S = 150
    c = synth.config1(seed=4, T=S)
    rng = np.random.default_rng(4)
    proj = synth.bf16r(rng.standard_normal((S, 8224)))
    proj[:, 8192:8208] = c["b"][0]
    proj[:, 8208:8224] = c["a"][0]
    st0 = (rng.standard_normal((1, 16, 128, 128)) * 0.02).astype(np.float32)
    y, st = gdn_chunked(bf16_dev(c["q"][0], dev), bf16_dev(c["k"][0], dev), bf16_dev(c["v"][0], dev), bf16_dev(proj, dev), f32_dev(c["A_log"], dev),
                        f32_dev(c["dt_bias"], dev), f32_dev(st0, dev))
    y_ref, s_ref = _oracle(c, S0=st0[0].astype(np.float64))
    assert y.shape == (S, 16, 128) and st.shape == (1, 16, 128, 128)
    assert orc.max_err_scaled(host(st[0]), s_ref) < STATE_TOL and orc.rel_l2(host(y), y_ref) < Y_REL_L2


def test_config4_ragged_batch_with_prefix_resume(dev):
    """Configuration 4 (seed 7): 16 sequences ~U[128, 4096] packed by cu_seqlens, every second one resuming from a cached state at a
    prefix that is a multiple of 64.  Oracle parity on four of the sequences; packing invariance on all."""
    c = synth.config4()
    q, k, v, lg, beta = _dev_case(dev, c)
    n = len(c["lengths"])
    idx = np.where(c["has_init"], np.arange(n), -1).astype(np.int32)
    y, s = gdn_chunked_varlen(q, k, v, lg, beta, i32_dev(c["cu_seqlens"], dev), init_state=f32_dev(c["init_state"], dev), init_idx=i32_dev(idx, dev))
    g = orc.compute_g(c["A_log"], c["a"], c["dt_bias"])
    bt = orc.beta_gate(c["b"])
    order = np.argsort(np.diff(c["cu_seqlens"]))
    for i in (order[0], order[1], order[2], order[n // 2]):
        a0, a1 = int(c["cu_seqlens"][i]), int(c["cu_seqlens"][i + 1])
        y_ref, s_ref = orc.gated_delta_rule(c["q"][a0:a1], c["k"][a0:a1], c["v"][a0:a1], g[a0:a1], bt[a0:a1], c["init_state"][i], np.float64)
        assert orc.max_err_scaled(host(s[i]), s_ref) < STATE_TOL
        assert orc.rel_l2(host(y[a0:a1]), y_ref) < Y_REL_L2
    assert bool(torch.isfinite(s).all()) and bool(torch.isfinite(y.float()).all())
    assert _lib.device_status() == 0


def test_rejects_bad_arguments(dev):
    z = torch.zeros((8, 16, 64), dtype=torch.bfloat16, device=dev)
    f = torch.zeros((8, 16), dtype=torch.float32, device=dev)
    with pytest.raises(ValueError):
        gdn_chunked_varlen(z, z, z, f, f, i32_dev([0, 8], dev))
    z = torch.zeros((8, 16, 128), dtype=torch.bfloat16, device=dev)
    with pytest.raises(ValueError):
        gdn_chunked_varlen(z, z, z, f, f, i32_dev([0, 8], dev), head_lo=3, head_hi=20)
