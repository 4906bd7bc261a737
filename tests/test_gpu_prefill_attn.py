"""GPU tests of the causal prefill attention (the scaled_dot_product_attention call of the reference's full-attention layer,
qwen35/model.py:148-169) against the oracle: ragged lengths, chunked continuation (pos > 0), both cache layouts, consistency with
the decode attention kernel on the same cache."""
import numpy as np
import pytest
import torch

from conftest import bf16_dev, host, i32_dev
from oracle import gdn_oracle as orc
from qwen_tailor_b200 import _lib, synth
from qwen_tailor_b200.attn_glue import prefill_attention
from qwen_tailor_b200.batch import attn_paged

pytestmark = pytest.mark.gpu
TOL_REL_L2 = 2e-3                                                      # bf16 outputs, the bound of the decode attention tests


def _qkv(S, T, seed, spread=1.0):
    rng = np.random.default_rng(seed)
    q = synth.bf16r(rng.standard_normal((S, 8, 256)) * spread)
    K = synth.bf16r(rng.standard_normal((2, T, 256)))
    V = synth.bf16r(rng.standard_normal((2, T, 256)))
    return q, K, V


@pytest.mark.parametrize("S,pos", [(1, 0), (5, 0), (31, 0), (32, 0), (33, 0), (64, 0), (100, 0), (257, 0), (2048, 0), (1, 77), (40, 24), (96, 1000), (300, 333)])
def test_prefill_attention_matches_the_oracle(dev, S, pos):
    q, K, V = _qkv(S, pos + S, seed=S * 7 + pos)
    o = prefill_attention(bf16_dev(q, dev), bf16_dev(K, dev), bf16_dev(V, dev), pos=pos, split=(S + pos) % 2 == 0)
    ref = orc.prefill_attention(q, K, V, pos)
    assert _lib.device_status() == 0
    got = host(o)
    assert orc.rel_l2(got, ref) <= TOL_REL_L2
    # the first query sees pos + 1 keys: a row-level check that the mask is where it belongs
    assert orc.rel_l2(got[0], ref[0]) <= 2 * TOL_REL_L2 and orc.rel_l2(got[-1], ref[-1]) <= 2 * TOL_REL_L2


def test_prefill_attention_peaked_scores(dev):
    """Scores with a spread of several hundred (log2 units): the running reference is raised many times, rows rescale the accumulator."""
    S = 200
    q, K, V = _qkv(S, S, seed=5, spread=12.0)
    o = prefill_attention(bf16_dev(q, dev), bf16_dev(K, dev), bf16_dev(V, dev))
    ref = orc.prefill_attention(q, K, V, 0)
    assert orc.rel_l2(host(o), ref) <= TOL_REL_L2 and _lib.device_status() == 0


def test_prefill_attention_cache_layouts_agree(dev):
    """Head-major [2, T, 256] (the reference's cache), the same inside a larger [1, 2, T_max, 256] buffer, and token-major [T, 2, 256]
    give the same bits."""
    S, pos = 130, 70
    q, K, V = _qkv(S, pos + S, seed=11)
    qd, Kd, Vd = bf16_dev(q, dev), bf16_dev(K, dev), bf16_dev(V, dev)
    o1 = prefill_attention(qd, Kd, Vd, pos=pos)
    big_k = torch.zeros((1, 2, 512, 256), dtype=torch.bfloat16, device=dev)
    big_v = torch.zeros_like(big_k)
    big_k[0, :, :pos + S] = Kd
    big_v[0, :, :pos + S] = Vd
    o2 = prefill_attention(qd, big_k, big_v, pos=pos)
    o3 = prefill_attention(qd, Kd.transpose(0, 1).contiguous(), Vd.transpose(0, 1).contiguous(), pos=pos)
    assert torch.equal(o1, o2) and torch.equal(o1, o3)


def test_chunked_prefill_equals_one_pass(dev):
    """Two chunks (pos = 0, then pos = S1 on the same cache) give the rows of the single pass: a row's result depends on its own
    keys only.  Bit-exact when the chunk boundary is a multiple of the 32-token query block, within the tolerance otherwise."""
    S = 320
    q, K, V = _qkv(S, S, seed=21)
    qd, Kd, Vd = bf16_dev(q, dev), bf16_dev(K, dev), bf16_dev(V, dev)
    full = prefill_attention(qd, Kd, Vd)
    for S1 in (128, 100):
        a = prefill_attention(qd[:S1].contiguous(), Kd, Vd, pos=0)
        b = prefill_attention(qd[S1:].contiguous(), Kd, Vd, pos=S1)
        got = torch.cat([a, b])
        if S1 % 32 == 0:
            assert torch.equal(got, full)
        else:
            assert orc.rel_l2(host(got), host(full).astype(np.float64)) <= TOL_REL_L2


def test_prefill_last_row_equals_decode_attention(dev):
    """The last query of a prefill chunk is what the decode kernel computes for one new token on the same cache (paged, 64-key pages)."""
    S = 500
    q, K, V = _qkv(S, S, seed=31)
    qd, Kd, Vd = bf16_dev(q, dev), bf16_dev(K, dev), bf16_dev(V, dev)
    o = prefill_attention(qd, Kd, Vd)
    n_pages = (S + 63) // 64
    kp = torch.zeros((n_pages, 2, 64, 256), dtype=torch.bfloat16, device=dev)
    vp = torch.zeros_like(kp)
    ctx = S - 1
    for t0 in range(0, ctx, 64):
        n = min(64, ctx - t0)
        kp[t0 // 64, :, :n] = Kd[:, t0:t0 + n]
        vp[t0 // 64, :, :n] = Vd[:, t0:t0 + n]
    table = i32_dev(np.arange(n_pages, dtype=np.int32)[None, :], dev)
    od = attn_paged(qd[S - 1:], Kd[:, S - 1].unsqueeze(0).contiguous(), Vd[:, S - 1].unsqueeze(0).contiguous(), kp, vp, table,
                    i32_dev(np.array([ctx], np.int32), dev), M=1, max_ctx=S)
    assert orc.rel_l2(host(od[0]), host(o[S - 1]).astype(np.float64)) <= TOL_REL_L2


def test_prefill_attention_rejects_bad_arguments(dev):
    q, K, V = _qkv(8, 8, seed=1)
    qd, Kd, Vd = bf16_dev(q, dev), bf16_dev(K, dev), bf16_dev(V, dev)
    with pytest.raises(ValueError):
        prefill_attention(qd, Kd, Vd, pos=4)                           # the cache is too short for pos + S
    with pytest.raises(ValueError):
        prefill_attention(qd, torch.zeros((3, 8, 256), dtype=torch.bfloat16, device=dev), torch.zeros((3, 8, 256), dtype=torch.bfloat16, device=dev))      # neither layout


def test_split_blocks_agree_with_unsplit_and_the_workspace_needs_no_reset(dev):
    """With a workspace the heaviest query blocks run as two blocks along the keys and are merged by the half that arrives last.
    Same result as the unsplit launch to rounding; the workspace's arrival counters carry an epoch tag, so one workspace -- filled with
    garbage at first -- serves call after call without being cleared."""
    from qwen_tailor_b200._lib import check, load, ptr, stream_ptr
    S = 1024
    q, K, V = _qkv(S, S, seed=41)
    qd, Kd, Vd = bf16_dev(q, dev), bf16_dev(K, dev), bf16_dev(V, dev)
    plain = prefill_attention(qd, Kd, Vd, split=False)
    lib = load()
    nbytes = int(lib.gqa_prefill_attn_workspace_bytes(S, 0))
    assert nbytes > 0 and int(lib.gqa_prefill_attn_workspace_bytes(4096, 0)) == 0       # more than one block per SM: never split
    ws = torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device=dev)
    outs = []
    for _ in range(3):
        out = torch.empty_like(qd)
        check(lib.gqa_prefill_attn(ptr(qd), ptr(Kd), ptr(Vd), ptr(out), S, 0, 256, S * 256, 256, S * 256, ptr(ws), nbytes, stream_ptr(dev)), "prefill")
        outs.append(out)
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    assert orc.rel_l2(host(outs[0]), host(plain).astype(np.float64)) <= 1e-3
    assert orc.rel_l2(host(outs[0]), orc.prefill_attention(q, K, V, 0)) <= TOL_REL_L2
    assert _lib.device_status() == 0
