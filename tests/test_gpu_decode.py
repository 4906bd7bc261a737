"""GPU parity of the recurrent decode / speculative-verify kernel against the CPU oracle, plus the reference's
hardware-independent bit contracts (tests/verify.py, tests/batch.py:42-100, tests/batch_spec.py:40-101 of the reference)."""
import numpy as np
import pytest
import torch

from conftest import bf16_dev, f32_dev, host, i32_dev
from oracle import gdn_oracle as orc
from qwen_tailor_b200 import _lib, synth
from qwen_tailor_b200.batch import deltanet_b
from qwen_tailor_b200.batch_spec import deltanet_bm
from qwen_tailor_b200.kernels import deltanet

pytestmark = pytest.mark.gpu

Y_REL_L2 = 2e-3          # bf16 outputs: rel-L2 and max|d|/max|ref| against the fp64 oracle rounded to bf16
STATE_TOL = 1e-4         # fp32 state: max|d|/max|ref|


def _case(dev, B, M, seed=1):
    c = synth.config2(B=B, seed=seed, M=M)
    t = dict(proj=bf16_dev(c["proj"], dev), conv=bf16_dev(c["conv"], dev), conv_w=bf16_dev(c["conv_w"], dev),
             A_log=f32_dev(c["A_log"], dev), dt_bias=f32_dev(c["dt_bias"], dev), state=f32_dev(c["state"], dev))
    return c, t


@pytest.mark.parametrize("M", [1, 3, 4])
def test_deltanet_matches_oracle(dev, M):
    c, t = _case(dev, 1, M)
    sel = i32_dev([0], dev)
    y, cs, st = deltanet(t["proj"], t["conv"], t["conv_w"], t["A_log"], t["dt_bias"], t["state"], sel)
    y_ref, y_un, cs_ref, st_ref = orc.deltanet(c["proj"], c["conv"][0], c["conv_w"], c["A_log"], c["dt_bias"], c["state"][0], np.float64)
    assert y.shape == (M, 2048) and cs.shape == (M, 3, 6144) and st.shape == (M, 16, 128, 128)
    assert np.array_equal(host(cs), cs_ref), "conv window snapshots are copies and must be bit-exact"
    assert orc.max_err_scaled(host(st), st_ref) < STATE_TOL
    assert orc.rel_l2(host(y), y_un) < Y_REL_L2
    assert orc.bf16_ulp_distance(host(y), y_ref).max() <= 1.0 + 1e-6 or orc.max_err_scaled(host(y), y_ref) < Y_REL_L2


def test_deltanet_start_snapshot_is_selected(dev):
    """The call starts from snapshot sel[0] of the state it is given (kernels.py:473-474)."""
    c, t = _case(dev, 3, 1, seed=4)                          # three snapshots, one token
    for s in range(3):
        y, cs, st = deltanet(t["proj"][:1], t["conv"], t["conv_w"], t["A_log"], t["dt_bias"], t["state"], i32_dev([s], dev))
        y1, cs1, st1 = deltanet(t["proj"][:1], t["conv"][s:s + 1], t["conv_w"], t["A_log"], t["dt_bias"], t["state"][s:s + 1], i32_dev([0], dev))
        assert torch.equal(y, y1) and torch.equal(cs, cs1) and torch.equal(st, st1)


def test_verify_m_equals_m_single_steps(dev):
    """verify(M=3) == 3 x verify(M=1), bit for bit: y, and snapshot 2 == the sequential final state."""
    c, t = _case(dev, 1, 3, seed=2)
    sel = i32_dev([0], dev)
    yB, csB, stB = deltanet(t["proj"], t["conv"], t["conv_w"], t["A_log"], t["dt_bias"], t["state"], sel)
    cs, st = t["conv"], t["state"]
    for j in range(3):
        y1, cs, st = deltanet(t["proj"][j:j + 1], cs, t["conv_w"], t["A_log"], t["dt_bias"], st, sel)
        assert torch.equal(y1[0], yB[j])
        assert torch.equal(st[0], stB[j]) and torch.equal(cs[0], csB[j])


def test_deltanet_b_equals_solo_rows(dev):
    """deltanet_b == solo deltanet per row (5 slots, ragged positions); in-place state; conv written to the other buffer;
    untouched slots untouched; the buffer that was read is preserved."""
    S, B = 6, 5
    rng = np.random.default_rng(11)
    slots = np.array([3, 0, 5, 1, 2], np.int32)
    pos = np.array([0, 1, 7, 100, 2047], np.int32)
    c = synth.config2(B=B, seed=11)
    proj = bf16_dev(synth.bf16r(rng.standard_normal((B, 8224)) * 2), dev)
    cv = synth.bf16r(rng.standard_normal((S + 1, 3, 6144)))
    ssm0 = (rng.standard_normal((S + 1, 16, 128, 128)) * 0.3).astype(np.float32)
    cp = synth.bf16r(rng.standard_normal(((S + 1) * 2, 3, 6144)))            # canary values everywhere
    for b in range(B):
        cp[slots[b] * 2 + (pos[b] & 1)] = cv[slots[b]]
    conv_pool, ssm_pool = bf16_dev(cp, dev), f32_dev(ssm0, dev)
    conv_w, A_log, dt_bias = bf16_dev(c["conv_w"], dev), f32_dev(c["A_log"], dev), f32_dev(c["dt_bias"], dev)
    y = deltanet_b(proj, conv_pool, conv_w, A_log, dt_bias, ssm_pool, i32_dev(slots, dev), i32_dev(pos, dev))
    sel0 = i32_dev([0], dev)
    cv_d, ssm0_d = bf16_dev(cv, dev), f32_dev(ssm0, dev)
    for b in range(B):
        s_ = int(slots[b])
        ry, rc, rs = deltanet(proj[b:b + 1], cv_d[s_:s_ + 1], conv_w, A_log, dt_bias, ssm0_d[s_:s_ + 1], sel0)
        assert torch.equal(y[b:b + 1], ry)
        assert torch.equal(ssm_pool[s_:s_ + 1], rs)
        assert torch.equal(conv_pool[s_ * 2 + ((int(pos[b]) & 1) ^ 1)][None], rc)
        assert np.array_equal(host(conv_pool[s_ * 2 + (int(pos[b]) & 1)]), cp[s_ * 2 + (int(pos[b]) & 1)])
    for s_ in (4, 6):
        assert np.array_equal(host(ssm_pool[s_]), ssm0[s_])
        assert np.array_equal(host(conv_pool[2 * s_:2 * s_ + 2]), cp[2 * s_:2 * s_ + 2])
    assert _lib.device_status() == 0


@pytest.mark.parametrize("B", [1, 16, 64])
def test_deltanet_b_matches_oracle_config2(dev, B):
    """Benchmark configuration 2 (B in {1, 16, 64}, seed 1): in-place pool step against the fp64 oracle."""
    c, t = _case(dev, B, 1)
    conv_pool = torch.zeros((B * 2, 3, 6144), dtype=torch.bfloat16, device=dev)
    pos = np.arange(B, dtype=np.int32) * 3
    for b in range(B):
        conv_pool[b * 2 + (pos[b] & 1)] = t["conv"][b]
    ssm_pool = t["state"].clone()
    y = deltanet_b(t["proj"], conv_pool, t["conv_w"], t["A_log"], t["dt_bias"], ssm_pool, i32_dev(np.arange(B), dev), i32_dev(pos, dev))
    check = range(B) if B <= 16 else range(0, B, 7)
    for b in check:
        y_ref, y_un, cs_ref, st_ref = orc.deltanet(c["proj"][b:b + 1], c["conv"][b], c["conv_w"], c["A_log"], c["dt_bias"], c["state"][b], np.float64)
        assert orc.max_err_scaled(host(ssm_pool[b]), st_ref[0]) < STATE_TOL
        assert orc.rel_l2(host(y[b]), y_un[0]) < Y_REL_L2
        assert np.array_equal(host(conv_pool[b * 2 + ((pos[b] & 1) ^ 1)]), cs_ref[0])


def test_deltanet_bm_equals_solo_verify(dev):
    """deltanet_bm == solo deltanet(M=3) per sequence: ragged entries / start snapshots / buffers, all M snapshots written,
    the buffer that was read preserved (tests/batch_spec.py:40-101 of the reference)."""
    NS, B, M = 5, 4, 3
    rng = np.random.default_rng(21)
    c = synth.config2(B=1, seed=21)
    sslots = np.array([2, 0, 4, 1], np.int32)
    sels = np.array([0, 2, 1, 2], np.int32)
    pars = np.array([0, 1, 1, 0], np.int32)
    proj = bf16_dev(synth.bf16r(rng.standard_normal((B * M, 8224)) * 2), dev)
    cp = synth.bf16r(rng.standard_normal(((NS + 1) * 2, M, 3, 6144)))
    sp = (rng.standard_normal((NS + 1, M, 16, 128, 128)) * 0.3).astype(np.float32)
    conv_pool, ssm_pool = bf16_dev(cp, dev), f32_dev(sp, dev)
    conv_w, A_log, dt_bias = bf16_dev(c["conv_w"], dev), f32_dev(c["A_log"], dev), f32_dev(c["dt_bias"], dev)
    y = deltanet_bm(proj, conv_pool, conv_w, A_log, dt_bias, ssm_pool, i32_dev(sslots, dev), i32_dev(sels, dev), i32_dev(pars, dev), M)
    cp_d, sp_d = bf16_dev(cp, dev), f32_dev(sp, dev)
    for b in range(B):
        e, sl, par = int(sslots[b]), int(sels[b]), int(pars[b])
        ry, rc, rs = deltanet(proj[b * M:(b + 1) * M], cp_d[e * 2 + par], conv_w, A_log, dt_bias, sp_d[e], i32_dev([sl], dev))
        assert torch.equal(y[b * M:(b + 1) * M], ry)
        assert torch.equal(ssm_pool[e], rs)
        assert torch.equal(conv_pool[e * 2 + (par ^ 1)], rc)
        assert np.array_equal(host(conv_pool[e * 2 + par]), cp[e * 2 + par])
    for e in (3, 5):
        assert np.array_equal(host(ssm_pool[e]), sp[e]) and np.array_equal(host(conv_pool[2 * e:2 * e + 2]), cp[2 * e:2 * e + 2])


def test_rollback_by_snapshot_index(dev):
    """Speculative rollback: after a verify of M tokens of which n are accepted, the next call with sel = n continues exactly
    as if only tokens 0..n had ever been fed (spec.py:40-63 of the reference)."""
    M = 4
    c, t = _case(dev, 1, 2 * M, seed=6)
    sel0 = i32_dev([0], dev)
    y1, cs1, st1 = deltanet(t["proj"][:M], t["conv"], t["conv_w"], t["A_log"], t["dt_bias"], t["state"], sel0)
    for n in range(M):
        yn, _, stn = deltanet(t["proj"][M:], cs1, t["conv_w"], t["A_log"], t["dt_bias"], st1, i32_dev([n], dev))
        # the same continuation from a run that only ever saw tokens 0..n
        y0, cs0, st0 = deltanet(t["proj"][:n + 1], t["conv"], t["conv_w"], t["A_log"], t["dt_bias"], t["state"], sel0)
        ya, _, sta = deltanet(t["proj"][M:], cs0[n:n + 1], t["conv_w"], t["A_log"], t["dt_bias"], st0[n:n + 1], sel0)
        assert torch.equal(yn, ya) and torch.equal(stn, sta)


def test_bad_slot_index_is_skipped_and_reported(dev):
    c, t = _case(dev, 2, 1)
    conv_pool = torch.zeros((4, 3, 6144), dtype=torch.bfloat16, device=dev)
    ssm_pool = t["state"].clone()
    before = ssm_pool.clone()
    _lib.device_status()
    deltanet_b(t["proj"], conv_pool, t["conv_w"], t["A_log"], t["dt_bias"], ssm_pool, i32_dev([0, 7], dev), i32_dev([0, 0], dev))
    assert _lib.device_status() == 1 and _lib.device_status() == 0
    assert torch.equal(ssm_pool[1], before[1]) and not torch.equal(ssm_pool[0], before[0])
