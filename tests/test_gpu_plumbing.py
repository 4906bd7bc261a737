"""GPU tests of the state plumbing around the kernels: the page-based prefix cache driven by the real prefill / attention kernels
(a hit == a prefill split at the checkpoint, bit for bit; decoding from a restored state never changes cached bits -- items 1, 2
and 4 of the reference's tests/prefix_cache.py), the plain <-> speculative pool moves (qwen35/serve.py:310-348), hrec, the
allocation-free attention wrapper, device-side index checks, and the B = 64, M = 4 verify shape."""
import numpy as np
import pytest
import torch

from conftest import bf16_dev, f32_dev, host, i32_dev
from qwen_tailor_b200 import _lib, synth
from qwen_tailor_b200.batch import Pools, attn_paged, attn_paged_static, deltanet_b, hrec
from qwen_tailor_b200.batch_spec import SpecPools, deltanet_bm
from qwen_tailor_b200.config import Cfg
from qwen_tailor_b200.gated_delta import gates
from qwen_tailor_b200.gdn_nax import gdn_chunked_varlen
from qwen_tailor_b200.kernels import deltanet
from qwen_tailor_b200.prefix_cache import PrefixCache

pytestmark = pytest.mark.gpu

N_LIN, N_FULL = 2, 1          # a cut-down layer stack: the plumbing does not depend on the layer count


def _prefill(dev, layers, t0, t1, state):
    """Run the GDN layers over tokens [t0, t1) from `state` (None = zeros) and append that range's K/V rows; returns the new state
    dict in the reference's form (dense K/V buffers of 512 rows)."""
    n = t1 - t0
    cu = i32_dev([0, n], dev)
    ssm, conv, ys = [], [], []
    for li, L in enumerate(layers["gdn"]):
        init = None if state is None else state["ssm"][li]
        y, s = gdn_chunked_varlen(L["q"][t0:t1].contiguous(), L["k"][t0:t1].contiguous(), L["v"][t0:t1].contiguous(), L["lg"][t0:t1].contiguous(),
                                  L["beta"][t0:t1].contiguous(), cu, init_state=init)
        ssm.append(s)
        conv.append(L["raw"][t1 - 3:t1][None].contiguous())
        ys.append(y)
    kv = []
    for li, A in enumerate(layers["attn"]):
        K = torch.zeros((1, 2, 512, 256), dtype=torch.bfloat16, device=dev)
        V = torch.zeros_like(K)
        if state is not None:
            K[:, :, :t0] = state["kv"][li][0][:, :, :t0]
            V[:, :, :t0] = state["kv"][li][1][:, :, :t0]
        K[0, :, t0:t1] = A["k"][t0:t1].transpose(0, 1)
        V[0, :, t0:t1] = A["v"][t0:t1].transpose(0, 1)
        kv.append((K, V))
    return {"kv": kv, "conv": conv, "ssm": ssm}, ys


def _layers(dev, T, seed):
    rng = np.random.default_rng(seed)
    out = {"gdn": [], "attn": []}
    for _ in range(N_LIN):
        A_log, dt_bias = synth.layer_params(rng)
        q, k, v, a, b = synth.gdn_tokens(rng, T)
        _, lg, beta = gates(bf16_dev(a, dev), bf16_dev(b, dev), f32_dev(A_log, dev), f32_dev(dt_bias, dev))
        out["gdn"].append(dict(q=bf16_dev(q, dev), k=bf16_dev(k, dev), v=bf16_dev(v, dev), lg=lg, beta=beta,
                               raw=bf16_dev(synth.bf16r(rng.standard_normal((T, 6144))), dev)))
    for _ in range(N_FULL):
        out["attn"].append(dict(k=bf16_dev(synth.bf16r(rng.standard_normal((T, 2, 256))), dev), v=bf16_dev(synth.bf16r(rng.standard_normal((T, 2, 256))), dev)))
    return out


def test_prefix_cache_hit_equals_split_prefill_and_never_aliases(dev):
    T, P1 = 320, 192                                               # the checkpoint sits on a chunk boundary (multiple of 64)
    toks = np.arange(7000, 7000 + T, dtype=np.int32)
    layers = _layers(dev, T, seed=31)
    pc = PrefixCache(budget_mb=256, page_size=64, kv_pages=32)
    # first request: prefill [0, P1), checkpoint, prefill the rest
    st1, _ = _prefill(dev, layers, 0, P1, None)
    node = pc.insert(None, toks, P1, st1)
    st_full, ys_full = _prefill(dev, layers, P1, T, st1)
    # second request with the same prefix: hit, restore, prefill only the suffix
    hit, split = pc.lookup(toks)
    assert hit is node and split == 0 and pc.last_hit == P1
    st_r, chain = pc.restore(hit, 512)
    assert [c.pos for c in chain] == [P1]
    for (K, V), (K0, V0) in zip(st_r["kv"], st1["kv"]):
        assert torch.equal(K, K0) and torch.equal(V, V0)
    st_hit, ys_hit = _prefill(dev, layers, P1, T, st_r)
    for a, b in zip(ys_hit, ys_full):
        assert torch.equal(a, b), "a hit equals the prefill that was split at the checkpoint, bit for bit"
    for a, b in zip(st_hit["ssm"], st_full["ssm"]):
        assert torch.equal(a, b)
    # ... and, the split being chunk-aligned, it also equals the unsplit prefill
    _, ys_one = _prefill(dev, layers, 0, T, None)
    for a, b in zip(ys_one, ys_full):
        assert torch.equal(a[P1:], b)
    # decoding from the restored state in place (slot pools) leaves the cached bits alone
    cfg = Cfg(layers=4, full_attn_interval=4)                       # 3 linear + 1 full: the pools take what they are given
    before_ssm, before_conv = hit.ssm.clone(), hit.conv.clone()
    pools = Pools(Cfg(), 2, 512, device=dev)
    pools.conv, pools.ssm, pools.K, pools.V = pools.conv[:N_LIN], pools.ssm[:N_LIN], pools.K[:N_FULL], pools.V[:N_FULL]
    pools.load(1, st_r, P1)
    c2 = synth.config2(B=1, seed=5)
    y = deltanet_b(bf16_dev(c2["proj"], dev), pools.conv[0], bf16_dev(c2["conv_w"], dev), f32_dev(c2["A_log"], dev), f32_dev(c2["dt_bias"], dev),
                   pools.ssm[0], i32_dev([1], dev), i32_dev([P1], dev))
    assert bool(torch.isfinite(y.float()).all()) and not torch.equal(pools.ssm[0][1], st_r["ssm"][0][0])
    st_r["ssm"][0].zero_()
    assert torch.equal(hit.ssm, before_ssm) and torch.equal(hit.conv, before_conv)
    again, _ = pc.restore(hit, 512)
    assert torch.equal(again["ssm"][0], st1["ssm"][0]) and torch.equal(again["conv"][1], st1["conv"][1])
    assert cfg.n_linear == 3 and _lib.device_status() == 0


def test_prefix_cache_paged_restore_feeds_the_attention_kernel(dev):
    """restore_paged gives page numbers that attn_paged reads directly: attention over the shared pages == attention over the dense
    K/V the checkpoint was made from; the appended row goes to the sequence's own copy of the last page."""
    T, P1 = 200, 150                                               # 150 = 2 full pages + 22 rows
    toks = np.arange(100, 100 + T, dtype=np.int32)
    layers = _layers(dev, T, seed=41)
    st1, _ = _prefill(dev, layers, 0, P1, None)
    pc = PrefixCache(budget_mb=256, page_size=64, kv_pages=16)
    node = pc.insert(None, toks, P1, st1)
    live, _ = pc.restore_paged(node)
    pool = pc.pool
    assert live["pages"][:2] == node.pages[:2] and live["pages"][2] != node.pages[2]
    rng = np.random.default_rng(3)
    q = bf16_dev(synth.bf16r(rng.standard_normal((1, 8, 256))), dev)
    kn = bf16_dev(synth.bf16r(rng.standard_normal((1, 2, 256))), dev)
    vn = bf16_dev(synth.bf16r(rng.standard_normal((1, 2, 256))), dev)
    cached_page = pool.K[0][node.pages[2]].clone()
    o_paged = attn_paged(q, kn, vn, pool.K[0], pool.V[0], i32_dev([live["pages"] + [0]], dev), i32_dev([P1], dev), M=1)
    # dense reference: the same attention over a one-page-per-sequence pool built from the dense buffers
    Kd, Vd = st1["kv"][0]
    o_dense = attn_paged(q, kn, vn, Kd.clone(), Vd.clone(), i32_dev([[0]], dev), i32_dev([P1], dev), M=1)
    assert torch.equal(o_paged, o_dense)
    tail = live["pages"][2]
    assert torch.equal(pool.K[0][tail, :, P1 - 128], kn[0]) and torch.equal(pool.K[0][node.pages[2]], cached_page)
    pc.release_pages(live["pages"])
    assert _lib.device_status() == 0


def test_spec_pools_enter_verify_leave_equals_plain_steps(dev):
    """A sequence moved into the snapshot pools, verified for M tokens and moved back at `sel` is in the state the plain in-place
    step reaches after sel + 1 tokens (qwen35/serve.py:310-348)."""
    M, slot, entry, pos = 3, 1, 2, 7
    c = synth.config2(B=1, seed=9, M=M)
    cfg = Cfg()
    pools, spec = Pools(cfg, 3, 64, device=dev), SpecPools(cfg, 3, 3, M, 64, device=dev)
    conv_w, A_log, dtb = bf16_dev(c["conv_w"], dev), f32_dev(c["A_log"], dev), f32_dev(c["dt_bias"], dev)
    proj = bf16_dev(c["proj"], dev)
    for i in range(cfg.n_linear):
        pools.ssm[i][slot] = f32_dev(c["state"][0], dev) * (1 + 0.1 * i)
        pools.conv[i][slot * 2 + (pos & 1)] = bf16_dev(c["conv"][0], dev)
    plain_ssm, plain_conv = [p.clone() for p in pools.ssm], [p.clone() for p in pools.conv]
    spec.enter(pools, slot, entry, pos)
    ys = [deltanet_bm(proj, spec.conv[i], conv_w, A_log, dtb, spec.ssm[i], i32_dev([entry], dev), i32_dev([0], dev), i32_dev([0], dev), M)
          for i in range(cfg.n_linear)]
    sel = 1                                                         # two tokens accepted
    spec.leave(pools, slot, entry, sel, 1, pos + sel + 1)           # the round wrote conv buffer 1
    for i in (0, 7, 17):
        p = pos
        for j in range(sel + 1):
            yj = deltanet_b(proj[j:j + 1], plain_conv[i], conv_w, A_log, dtb, plain_ssm[i], i32_dev([slot], dev), i32_dev([p], dev))
            assert torch.equal(yj[0], ys[i][j])
            p += 1
        assert torch.equal(pools.ssm[i][slot], plain_ssm[i][slot])
        assert torch.equal(pools.conv[i][slot * 2 + (p & 1)], plain_conv[i][slot * 2 + (p & 1)])
    assert _lib.device_status() == 0


def test_hrec_scatters_rows(dev):
    hist = torch.zeros((4, 16, 1024), dtype=torch.bfloat16, device=dev)
    Hn = torch.randn((3, 1024), device=dev).to(torch.bfloat16)
    slots, pos = i32_dev([2, 0, 3], dev), i32_dev([5, 0, 15], dev)
    out = hrec(hist, Hn, slots, pos)
    assert out is hist
    for b, (s, p) in enumerate(((2, 5), (0, 0), (3, 15))):
        assert torch.equal(hist[s, p], Hn[b])
    assert int((hist != 0).any(-1).sum()) == 3, "only the three addressed rows change"
    assert _lib.device_status() == 0
    # an odd width takes the element-wise path; a bad slot or position skips its row and is reported
    hist2 = torch.zeros((4, 16, 1001), dtype=torch.bfloat16, device=dev)
    Hn2 = torch.randn((3, 1001), device=dev).to(torch.bfloat16)
    hrec(hist2, Hn2, i32_dev([1, 9, 2], dev), i32_dev([3, 0, 16], dev))
    assert torch.equal(hist2[1, 3], Hn2[0]) and int((hist2 != 0).any(-1).sum()) == 1
    assert _lib.device_status() == 1 and _lib.device_status() == 0


def test_attn_paged_static_wrapper_equals_attn_paged(dev):
    rng = np.random.default_rng(8)
    a = synth.attn_case(rng, [700, 64, 1500], 2, 64)
    args = [bf16_dev(a[n], dev) for n in ("q", "k_new", "v_new")]
    kp, vp = bf16_dev(a["k_pages"], dev), bf16_dev(a["v_pages"], dev)
    bt, cl = i32_dev(a["block_table"], dev), i32_dev(a["ctx_len"], dev)
    o1 = attn_paged(*args, kp.clone(), vp.clone(), bt, cl, M=2)
    kp2, vp2 = kp.clone(), vp.clone()
    o2 = attn_paged_static(*args, kp2, vp2, bt, cl, M=2)
    assert torch.equal(o1, o2)
    with pytest.raises(ValueError):
        attn_paged_static(torch.zeros((257, 8, 256), dtype=torch.bfloat16, device=dev), torch.zeros((257, 2, 256), dtype=torch.bfloat16, device=dev),
                          torch.zeros((257, 2, 256), dtype=torch.bfloat16, device=dev), kp2, vp2, torch.zeros((257, 1), dtype=torch.int32, device=dev),
                          torch.zeros(257, dtype=torch.int32, device=dev), M=1)
    assert _lib.device_status() == 0


@pytest.mark.parametrize("page", [16, 64])
def test_corrupt_page_table_entry_is_reported(dev, page):
    """A block-table entry outside the pool, in the middle of a valid context: both load paths (gathered copies for 16-row pages,
    tensor-map copies for 64-row pages) report it through the status word, read page 0 instead, and fault nothing."""
    rng = np.random.default_rng(9)
    a = synth.attn_case(rng, [300, 40], 1, page)
    bt = a["block_table"].copy()
    bt[0, 2] = 10 ** 6
    o = attn_paged(bf16_dev(a["q"], dev), bf16_dev(a["k_new"], dev), bf16_dev(a["v_new"], dev), bf16_dev(a["k_pages"], dev), bf16_dev(a["v_pages"], dev),
                   i32_dev(bt, dev), i32_dev(a["ctx_len"], dev), M=1)
    torch.cuda.synchronize()
    assert _lib.device_status() == 1
    assert bool(torch.isfinite(o.float()).all())
    # the other sequence is unaffected
    o_ok = attn_paged(bf16_dev(a["q"], dev), bf16_dev(a["k_new"], dev), bf16_dev(a["v_new"], dev), bf16_dev(a["k_pages"], dev), bf16_dev(a["v_pages"], dev),
                      i32_dev(a["block_table"], dev), i32_dev(a["ctx_len"], dev), M=1)
    assert torch.equal(o[1], o_ok[1]) and _lib.device_status() == 0


def test_verify_64_sequences_4_tokens_equal_solo_rows(dev):
    """deltanet_bm at B = 64, M = 4 (the launch splits heads across blocks at this size): every checked sequence equals the solo
    verify on its rows, bit for bit, with ragged start snapshots and buffers."""
    B, M = 64, 4
    rng = np.random.default_rng(64)
    c = synth.config2(B=B, seed=64, M=M)
    proj, conv_w = bf16_dev(c["proj"], dev), bf16_dev(c["conv_w"], dev)
    A_log, dtb = f32_dev(c["A_log"], dev), f32_dev(c["dt_bias"], dev)
    sels = rng.integers(0, M, B).astype(np.int32)
    pars = rng.integers(0, 2, B).astype(np.int32)
    sslots = rng.permutation(B).astype(np.int32)
    ssm = (torch.randn((B + 1, M, 16, 128, 128), device=dev) * 0.02)
    conv = torch.randn(((B + 1) * 2, M, 3, 6144), device=dev).to(torch.bfloat16)
    ssm0, conv0 = ssm.clone(), conv.clone()
    y = deltanet_bm(proj, conv, conv_w, A_log, dtb, ssm, i32_dev(sslots, dev), i32_dev(sels, dev), i32_dev(pars, dev), M)
    sel0 = i32_dev([0], dev)
    for b in range(0, B, 9):
        e, s, p = int(sslots[b]), int(sels[b]), int(pars[b])
        yb, cb, sb = deltanet(proj[b * M:(b + 1) * M], conv0[e * 2 + p, s][None].contiguous(), conv_w, A_log, dtb, ssm0[e, s][None].contiguous(), sel0)
        assert torch.equal(y[b * M:(b + 1) * M], yb) and torch.equal(ssm[e], sb) and torch.equal(conv[e * 2 + (p ^ 1)], cb)
        assert torch.equal(conv[e * 2 + p], conv0[e * 2 + p]), "the buffer that was read is preserved"
    assert torch.equal(ssm[B], ssm0[B]) and _lib.device_status() == 0


def test_paged_pools_serve_decode_steps_and_share_pages_with_the_prefix_cache(dev):
    """PagedPools (K/V of the slots in the prefix cache's page pool) against the reference-layout Pools: the same attention and
    delta-rule outputs over several decode steps; a checkpoint taken from a slot shares the slot's full pages, a hit hands another
    slot those pages without copying K/V, and the two sequences then diverge on private pages."""
    from qwen_tailor_b200.batch import attn_b
    from qwen_tailor_b200.paged_pools import PagedPools
    cfg = Cfg()
    Lmax, lens = 256, [150, 70]
    dense = Pools(cfg, 3, Lmax, device=dev)
    paged = PagedPools(cfg, 3, Lmax, n_pages=24, device=dev)
    g = torch.Generator(device=dev); g.manual_seed(5)
    rnb = lambda *s: torch.randn(s, generator=g, device=dev).to(torch.bfloat16)
    for slot, pos in enumerate(lens):
        st = {"kv": [], "conv": [rnb(1, 3, 6144) for _ in range(cfg.n_linear)],
              "ssm": [torch.randn((1, 16, 128, 128), generator=g, device=dev) * 0.02 for _ in range(cfg.n_linear)]}
        for _ in range(cfg.n_full):
            K, V = torch.zeros((1, 2, Lmax, 256), dtype=torch.bfloat16, device=dev), torch.zeros((1, 2, Lmax, 256), dtype=torch.bfloat16, device=dev)
            K[:, :, :pos], V[:, :, :pos] = rnb(1, 2, pos, 256), rnb(1, 2, pos, 256)
            st["kv"].append((K, V))
        dense.load(slot, st, pos)
        paged.admit(slot, st, pos)
    slots = i32_dev([0, 1], dev)
    c = synth.config2(B=2, seed=3, M=1)
    cw, A_log, dtb = bf16_dev(c["conv_w"], dev), f32_dev(c["A_log"], dev), f32_dev(c["dt_bias"], dev)
    cur = list(lens)
    for step in range(3):
        ctx = i32_dev(cur, dev)
        for s_ in range(2):
            paged.reserve(s_, cur[s_] + 1)
        q, kn, vn = rnb(2, 8, 256), rnb(2, 2, 256), rnb(2, 2, 256)
        o_d = attn_b(q, kn, vn, dense.K[1], dense.V[1], slots, ctx, M=1)
        o_p = paged.attn(1, q, kn, vn, slots, ctx, M=1)
        assert torch.equal(o_d, o_p)
        proj = rnb(2, 8224)
        y_d = deltanet_b(proj, dense.conv[2], cw, A_log, dtb, dense.ssm[2], slots, ctx)
        y_p = paged.deltanet(2, proj, cw, A_log, dtb, slots, ctx)
        assert torch.equal(y_d, y_p)
        for s_ in range(2):
            cur[s_] += 1
            paged.advance(s_, 1)
    # ---- a checkpoint of slot 0 (153 tokens = 2 full pages + 25 rows) shares its full pages; a hit gives them to slot 2 ----
    pc = PrefixCache(budget_mb=256, kv_pages=paged.pages)
    toks = np.arange(500, 500 + cur[0], dtype=np.int32)
    node = pc.insert(None, toks, cur[0], paged.checkpoint_state(0))
    assert node.pages[:2] == paged.owned[0][:2] and all(paged.pages.refs[p] == 2 for p in node.pages[:2])
    hit, _ = pc.lookup(np.concatenate([toks, [7, 8]]))
    assert hit is node
    live, _ = pc.restore_paged(hit)
    paged.admit_paged(2, live, cur[0])
    assert paged.owned[2][:2] == paged.owned[0][:2] and paged.owned[2][2] != paged.owned[0][2]
    both = i32_dev([0, 2], dev)
    ctx = i32_dev([cur[0], cur[0]], dev)
    paged.reserve(0, cur[0] + 1); paged.reserve(2, cur[0] + 1)
    q1, kn1, vn1 = rnb(1, 8, 256), rnb(2, 2, 256), rnb(1, 2, 256)
    q2 = torch.cat([q1, q1])
    o = paged.attn(0, q2, kn1, torch.cat([vn1, vn1]), both, ctx, M=1)
    # same cached keys, same query; the appended key differs, so the outputs differ only through the new row -- and each slot wrote
    # its own page: the checkpoint's copy and the other slot's page are untouched
    row = cur[0] % 64
    assert torch.equal(paged.pages.K[0][paged.owned[0][2], :, row], kn1[0]) and torch.equal(paged.pages.K[0][paged.owned[2][2], :, row], kn1[1])
    assert not torch.equal(o[0], o[1])
    o_again = paged.attn(0, q2, torch.cat([kn1[:1], kn1[:1]]), torch.cat([vn1, vn1]), both, ctx, M=1)
    assert torch.equal(o_again[0], o_again[1]) and torch.equal(o_again[0], o[0])
    paged.release(0); paged.release(2); paged.release(1)
    pc.clear()
    assert paged.pages.available() == paged.pages.n_pages - 1
    assert _lib.device_status() == 0
