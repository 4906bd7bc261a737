"""Full-size runs of the benchmark configurations, checked through size-independent properties (the oracle would need minutes):
split == resume for a T = 8192 prefill, the whole speculative-verify step of configuration 5 with rollback at random accept
lengths, and decode of 64 sequences against the per-row solo kernel."""
import numpy as np
import pytest
import torch

from conftest import bf16_dev, f32_dev, host, i32_dev
from oracle import gdn_oracle as orc
from qwen_tailor_b200 import _lib, synth
from qwen_tailor_b200.batch import attn_paged
from qwen_tailor_b200.batch_spec import accept_length, deltanet_bm
from qwen_tailor_b200.gated_delta import gates
from qwen_tailor_b200.gdn_nax import gdn_chunked_varlen
from qwen_tailor_b200.kernels import deltanet

pytestmark = pytest.mark.gpu


def test_prefill_8192_split_equals_resume_and_tail_matches_oracle(dev):
    """Configuration 3 at T = 8192 (layer seed 100): one pass == three resumed passes bit for bit; the last 192 tokens, restarted
    from the kernel's own state at 8000, match the fp64 oracle; everything is finite."""
    T = 8192
    c = synth.config3_layer(0, T)
    q, k, v = (bf16_dev(c[n], dev) for n in "qkv")
    _, lg, beta = gates(bf16_dev(c["a"], dev), bf16_dev(c["b"], dev), f32_dev(c["A_log"], dev), f32_dev(c["dt_bias"], dev))
    y, s = gdn_chunked_varlen(q, k, v, lg, beta, i32_dev([0, T], dev))
    assert bool(torch.isfinite(y.float()).all()) and bool(torch.isfinite(s).all())
    st, ys = None, []
    for a0, a1 in ((0, 2048), (2048, 8000 - 8000 % 64), (8000 - 8000 % 64, T)):
        yi, st = gdn_chunked_varlen(q[a0:a1].contiguous(), k[a0:a1].contiguous(), v[a0:a1].contiguous(), lg[a0:a1].contiguous(),
                                    beta[a0:a1].contiguous(), i32_dev([0, a1 - a0], dev), init_state=st)
        ys.append(yi)
    assert torch.equal(torch.cat(ys), y) and torch.equal(st, s)
    P = 8000 - 8000 % 64
    _, sP = gdn_chunked_varlen(q[:P].contiguous(), k[:P].contiguous(), v[:P].contiguous(), lg[:P].contiguous(), beta[:P].contiguous(), i32_dev([0, P], dev))
    g = orc.compute_g(c["A_log"], c["a"][P:], c["dt_bias"])
    y_ref, s_ref = orc.gated_delta_rule(c["q"][P:], c["k"][P:], c["v"][P:], g, orc.beta_gate(c["b"][P:]), host(sP[0]).astype(np.float64))
    assert orc.max_err_scaled(host(s[0]), s_ref) < 1e-4 and orc.rel_l2(host(y[P:]), y_ref) < 2e-3


def test_config5_verify_step_with_rollback(dev):
    """Configuration 5 (seed 11): B = 16 sequences verify K = 4 draft tokens through a GDN layer (snapshot pools, in place) and a
    full-attention layer (paged cache, ctx ~ U[1024, 8192]); then every sequence rolls back to a random accept length 0..4 and the
    next round, started from the chosen snapshot, equals a run that only ever saw the accepted tokens."""
    B, M = 16, 4
    ctx, accept = synth.config5_shapes()
    rng = np.random.default_rng(11)
    c = synth.config2(B=B, seed=11, M=2 * M)
    proj1 = bf16_dev(c["proj"].reshape(B, 2 * M, -1)[:, :M].reshape(B * M, -1), dev)
    proj2 = bf16_dev(c["proj"].reshape(B, 2 * M, -1)[:, M:].reshape(B * M, -1), dev)
    conv_w, A_log, dtb = bf16_dev(c["conv_w"], dev), f32_dev(c["A_log"], dev), f32_dev(c["dt_bias"], dev)
    NS = B
    conv_pool = torch.zeros(((NS + 1) * 2, M, 3, 6144), dtype=torch.bfloat16, device=dev)
    ssm_pool = torch.zeros((NS + 1, M, 16, 128, 128), dtype=torch.float32, device=dev)
    conv_pool[0:2 * B:2, 0] = bf16_dev(c["conv"], dev)                       # entry b, buffer 0, snapshot 0 = the incoming state
    ssm_pool[:B, 0] = f32_dev(c["state"], dev)
    ss = i32_dev(np.arange(B), dev)
    y1 = deltanet_bm(proj1, conv_pool, conv_w, A_log, dtb, ssm_pool, ss, i32_dev(np.zeros(B), dev), i32_dev(np.zeros(B), dev), M)
    assert y1.shape == (B * M, 2048) and bool(torch.isfinite(ssm_pool).all())
    # acceptance: toks[:, 1:] are the drafts, ids the verified tokens; construct ids so that n_new == accept - 1 (accept >= 1)
    toks = rng.integers(0, 1000, (B, M + 1)).astype(np.int32)
    ids = toks[:, 1:].copy()
    for b in range(B):
        if accept[b] < M:
            ids[b, accept[b]] += 1                                           # first mismatch right after the accepted drafts
    n_new = accept_length(torch.from_numpy(toks).to(dev), torch.from_numpy(np.concatenate([ids, ids[:, :1]], 1)).to(dev))
    assert np.array_equal(host(n_new), orc.accept_length(toks, np.concatenate([ids, ids[:, :1]], 1))) and np.array_equal(host(n_new), accept)
    # rollback: accept a >= 1 tokens -> continue from snapshot a - 1; a == 0 -> keep the incoming state (a fresh pool entry)
    sel = np.maximum(accept - 1, 0).astype(np.int32)
    keep = accept == 0
    ssm2, conv2 = ssm_pool.clone(), conv_pool.clone()
    for b in np.where(keep)[0]:
        ssm2[b, 0] = f32_dev(c["state"][b], dev)
        conv2[2 * b + 1, 0] = bf16_dev(c["conv"][b], dev)
    y2 = deltanet_bm(proj2, conv2, conv_w, A_log, dtb, ssm2, ss, i32_dev(sel, dev), i32_dev(np.ones(B), dev), M)
    sel0 = i32_dev([0], dev)
    for b in (0, 3, 7, 15):
        a_ = int(accept[b])
        cs, st = bf16_dev(c["conv"][b:b + 1], dev), f32_dev(c["state"][b:b + 1], dev)
        if a_ > 0:
            _, csa, sta = deltanet(proj1[b * M:b * M + a_], cs, conv_w, A_log, dtb, st, sel0)
            cs, st = csa[-1:].contiguous(), sta[-1:].contiguous()
        yb, _, stb = deltanet(proj2[b * M:(b + 1) * M], cs, conv_w, A_log, dtb, st, sel0)
        assert torch.equal(y2[b * M:(b + 1) * M], yb) and torch.equal(ssm2[b], stb)
    # the attention half of the step: M rows per sequence over the paged cache
    page = 64
    a5 = synth.attn_case(rng, ctx, M, page)
    o = attn_paged(bf16_dev(a5["q"], dev), bf16_dev(a5["k_new"], dev), bf16_dev(a5["v_new"], dev), bf16_dev(a5["k_pages"], dev),
                   bf16_dev(a5["v_pages"], dev), i32_dev(a5["block_table"], dev), i32_dev(a5["ctx_len"], dev), M=M)
    for b in (int(np.argmin(ctx)), int(np.argmax(ctx))):
        pages = a5["block_table"][b]
        n = int(ctx[b])
        gather = lambda Pg: np.concatenate([Pg[p] for p in pages], axis=1)[:, :n]
        rsl = slice(b * M, (b + 1) * M)
        ref = orc.attn_rows(a5["q"][rsl], a5["k_new"][rsl], a5["v_new"][rsl], gather(a5["k_pages"]), gather(a5["v_pages"]))
        assert orc.rel_l2(host(o[rsl]), ref) < 2e-3
    assert _lib.device_status() == 0


def test_decode_64_rows_equal_solo_rows(dev):
    """Configuration 2 at B = 64: every row of the batched in-place step equals the solo kernel on that row, bit for bit."""
    from qwen_tailor_b200.batch import deltanet_b
    B = 64
    c = synth.config2(B=B, seed=1)
    proj, conv_w = bf16_dev(c["proj"], dev), bf16_dev(c["conv_w"], dev)
    A_log, dtb = f32_dev(c["A_log"], dev), f32_dev(c["dt_bias"], dev)
    conv_pool = torch.zeros(((B + 1) * 2, 3, 6144), dtype=torch.bfloat16, device=dev)
    conv_pool[0:2 * B:2] = bf16_dev(c["conv"], dev)
    ssm_pool = torch.cat([f32_dev(c["state"], dev), torch.zeros((1, 16, 128, 128), device=dev)])
    slots = torch.randperm(B, device=dev).to(torch.int32)
    ref_state, ref_conv = ssm_pool.clone(), conv_pool.clone()
    y = deltanet_b(proj, conv_pool, conv_w, A_log, dtb, ssm_pool, slots, torch.zeros(B, dtype=torch.int32, device=dev))
    sel0 = i32_dev([0], dev)
    for b in range(0, B, 5):
        s_ = int(slots[b])
        yb, cb, sb = deltanet(proj[b:b + 1], ref_conv[2 * s_:2 * s_ + 1], conv_w, A_log, dtb, ref_state[s_:s_ + 1], sel0)
        assert torch.equal(y[b:b + 1], yb) and torch.equal(ssm_pool[s_:s_ + 1], sb) and torch.equal(conv_pool[2 * s_ + 1][None], cb)
    assert torch.equal(ssm_pool[B], ref_state[B])
