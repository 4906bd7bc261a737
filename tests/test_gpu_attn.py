"""GPU parity of the GQA decode attention (slot pool and paged cache) and of the strided copies / pools."""
import numpy as np
import pytest
import torch

from conftest import bf16_dev, f32_dev, host, i32_dev
from oracle import gdn_oracle as orc
from qwen_tailor_b200 import Cfg, _lib, synth
from qwen_tailor_b200.batch import Pools, attn_b, attn_paged, blit

pytestmark = pytest.mark.gpu

O_TOL = 4e-3             # bf16 output against the fp64 oracle: max|d| / max|ref| (one bf16 rounding = 2^-8 relative)
O_REL_L2 = 2e-3


def _check_rows(o, q, kn, vn, k_ctx, v_ctx, M):
    ref = orc.attn_rows(q, kn, vn, k_ctx, v_ctx)
    got = host(o)
    assert orc.rel_l2(got, ref) < O_REL_L2, orc.rel_l2(got, ref)
    assert orc.max_err_scaled(got, ref) < O_TOL


@pytest.mark.parametrize("M", [1, 3])
def test_attn_b_slot_pool(dev, M):
    """attn_b over the reference's slot pool layout: positions {0,1,31,32,300,1023-M+1}, GQA 4:1, append at pos, every other row of
    the pool untouched (tests/batch.py:70-100, tests/batch_spec.py:85-98 of the reference)."""
    S, Lmax, H, KV, D = 6, 1024, 8, 2, 256
    rng = np.random.default_rng(11)
    Kp = synth.bf16r(rng.standard_normal((S + 1, KV, Lmax, D)))
    Vp = synth.bf16r(rng.standard_normal((S + 1, KV, Lmax, D)))
    slots = np.array([3, 0, 5, 1, 2, 4], np.int32)
    pos = np.array([0, 1, 31, 32, 300, Lmax - M], np.int32)
    B = len(slots)
    q = synth.bf16r(rng.standard_normal((B * M, H, D)))
    kn = synth.bf16r(rng.standard_normal((B * M, KV, D)))
    vn = synth.bf16r(rng.standard_normal((B * M, KV, D)))
    Kd, Vd = bf16_dev(Kp, dev), bf16_dev(Vp, dev)
    o = attn_b(bf16_dev(q, dev), bf16_dev(kn, dev), bf16_dev(vn, dev), Kd, Vd, i32_dev(slots, dev), i32_dev(pos, dev), M=M)
    assert o.shape == (B * M, H, D) and o.dtype == torch.bfloat16
    Kh, Vh = host(Kd), host(Vd)
    for b in range(B):
        s_, p = int(slots[b]), int(pos[b])
        r = slice(b * M, (b + 1) * M)
        _check_rows(o[r], q[r], kn[r], vn[r], Kp[s_, :, :p], Vp[s_, :, :p], M)
        for j in range(M):
            assert np.array_equal(Kh[s_, :, p + j], kn[b * M + j]) and np.array_equal(Vh[s_, :, p + j], vn[b * M + j])
        assert np.array_equal(Kh[s_, :, :p], Kp[s_, :, :p]) and np.array_equal(Kh[s_, :, p + M:], Kp[s_, :, p + M:])
        assert np.array_equal(Vh[s_, :, :p], Vp[s_, :, :p]) and np.array_equal(Vh[s_, :, p + M:], Vp[s_, :, p + M:])
    assert np.array_equal(Kh[6], Kp[6]) and np.array_equal(Vh[6], Vp[6])
    assert _lib.device_status() == 0


@pytest.mark.parametrize("M,page_size,lo,hi", [(1, 16, 1, 700), (4, 64, 1024, 3000), (2, 128, 0, 5)])
def test_attn_paged_ragged(dev, M, page_size, lo, hi):
    """Paged cache, shuffled block table, ragged contexts (benchmark configuration 5 draws ctx ~ U[1024, 8192], M = 4)."""
    rng = np.random.default_rng(5 + M)
    ctx = rng.integers(lo, hi + 1, 7)
    ctx[0] = lo
    c = synth.attn_case(rng, ctx, M, page_size)
    Kd, Vd = bf16_dev(c["k_pages"], dev), bf16_dev(c["v_pages"], dev)
    o = attn_paged(bf16_dev(c["q"], dev), bf16_dev(c["k_new"], dev), bf16_dev(c["v_new"], dev), Kd, Vd, i32_dev(c["block_table"], dev),
                   i32_dev(c["ctx_len"], dev), M=M)
    Kh, Vh = host(Kd), host(Vd)
    touched = np.zeros(c["k_pages"].shape[:3], bool).transpose(0, 2, 1)          # [page, row, kv]
    for b in range(len(ctx)):
        n = int(ctx[b])
        pages = c["block_table"][b]
        gather = lambda Pg: np.concatenate([Pg[p] for p in pages], axis=1)[:, :n]  # [KV, n, D]
        r = slice(b * M, (b + 1) * M)
        _check_rows(o[r], c["q"][r], c["k_new"][r], c["v_new"][r], gather(c["k_pages"]), gather(c["v_pages"]), M)
        for j in range(M):
            pg, row = pages[(n + j) // page_size], (n + j) % page_size
            assert np.array_equal(Kh[pg, :, row], c["k_new"][b * M + j]) and np.array_equal(Vh[pg, :, row], c["v_new"][b * M + j])
            touched[pg, row] = True
    keep = ~touched.transpose(0, 2, 1)
    assert np.array_equal(Kh[keep], c["k_pages"][keep]) and np.array_equal(Vh[keep], c["v_pages"][keep])
    assert _lib.device_status() == 0


def test_attn_long_context_many_splits(dev):
    """One long sequence (8192 keys) forces the split-KV path with many splits; a short neighbour uses one."""
    rng = np.random.default_rng(9)
    c = synth.attn_case(rng, [8192, 40], 4, 64)
    o = attn_paged(bf16_dev(c["q"], dev), bf16_dev(c["k_new"], dev), bf16_dev(c["v_new"], dev), bf16_dev(c["k_pages"], dev),
                   bf16_dev(c["v_pages"], dev), i32_dev(c["block_table"], dev), i32_dev(c["ctx_len"], dev), M=4)
    for b, n in enumerate((8192, 40)):
        pages = c["block_table"][b]
        gather = lambda Pg: np.concatenate([Pg[p] for p in pages], axis=1)[:, :n]
        r = slice(b * 4, (b + 1) * 4)
        _check_rows(o[r], c["q"][r], c["k_new"][r], c["v_new"][r], gather(c["k_pages"]), gather(c["v_pages"]), 4)


def test_attn_rejects_unsupported(dev):
    z = lambda *s: torch.zeros(s, dtype=torch.bfloat16, device=dev)
    with pytest.raises(ValueError):
        attn_b(z(1, 8, 128), z(1, 2, 128), z(1, 2, 128), z(2, 2, 64, 128), z(2, 2, 64, 128), i32_dev([0], dev), i32_dev([0], dev))
    with pytest.raises(ValueError):
        attn_b(z(5, 8, 256), z(5, 2, 256), z(5, 2, 256), z(2, 2, 64, 256), z(2, 2, 64, 256), i32_dev([0], dev), i32_dev([0], dev), M=5)


def test_bad_page_index_is_reported(dev):
    rng = np.random.default_rng(1)
    c = synth.attn_case(rng, [20], 1, 16)
    table = c["block_table"].copy()
    table[0, 0] = 9999
    _lib.device_status()
    attn_paged(bf16_dev(c["q"], dev), bf16_dev(c["k_new"], dev), bf16_dev(c["v_new"], dev), bf16_dev(c["k_pages"], dev),
               bf16_dev(c["v_pages"], dev), i32_dev(table, dev), i32_dev([40], dev), M=1)     # context beyond the table
    assert _lib.device_status() == 1


def test_blit_and_pools_round_trip(dev):
    """blit semantics (batch.py:367-372) with aligned and unaligned offsets; Pools.load / read round trip (tests/batch.py:102-112)."""
    rng = np.random.default_rng(3)
    for dt, n, d0, s0, ny, ds, ss in ((torch.float32, 1000, 8, 16, 3, 2048, 1024), (torch.bfloat16, 77, 3, 5, 4, 100, 90),
                                      (torch.bfloat16, 6144 * 3, 6144 * 3 * 5, 0, 1, 0, 0), (torch.float32, 5, 1, 2, 1, 0, 0)):
        src = torch.from_numpy(rng.standard_normal(8192 * 4).astype(np.float32)).to(dev).to(dt)
        dst = torch.from_numpy(rng.standard_normal(8192 * 16).astype(np.float32)).to(dev).to(dt)
        want = dst.clone()
        for y in range(ny):
            want[d0 + y * ds:d0 + y * ds + n] = src[s0 + y * ss:s0 + y * ss + n]
        blit(dst, src, n, d0, s0, ny, ds, ss)
        assert torch.equal(dst, want)
    cfg = Cfg()
    P = Pools(cfg, 3, 256, device=dev)
    pos = 77
    st = {"conv": [bf16_dev(synth.bf16r(rng.standard_normal((1, 3, 6144))), dev) for _ in range(18)],
          "ssm": [f32_dev(rng.standard_normal((1, 16, 128, 128)), dev) for _ in range(18)],
          "kv": [(bf16_dev(synth.bf16r(rng.standard_normal((1, 2, 128, 256))), dev), bf16_dev(synth.bf16r(rng.standard_normal((1, 2, 128, 256))), dev))
                 for _ in range(6)]}
    P.load(2, st, pos)
    back = P.read(2, pos, 128)
    assert all(torch.equal(a, b) for a, b in zip(back["ssm"], st["ssm"])) and all(torch.equal(a, b) for a, b in zip(back["conv"], st["conv"]))
    assert all(torch.equal(a[0][:, :, :pos], b[0][:, :, :pos]) and torch.equal(a[1][:, :, :pos], b[1][:, :, :pos]) for a, b in zip(back["kv"], st["kv"]))
    assert all(float(P.ssm[i][0].abs().sum()) == 0 and float(P.ssm[i][3].abs().sum()) == 0 for i in range(18))
    assert P.nbytes() == 4 * Pools.slot_bytes(cfg, 256)


def _check_case(dev, c, ctx, M, page_size, o):
    for b in range(len(ctx)):
        n = int(ctx[b])
        pages = c["block_table"][b]
        gather = lambda Pg: np.concatenate([Pg[p] for p in pages], axis=1)[:, :n]
        r = slice(b * M, (b + 1) * M)
        _check_rows(o[r], c["q"][r], c["k_new"][r], c["v_new"][r], gather(c["k_pages"]), gather(c["v_pages"]), M)


@pytest.mark.parametrize("ctx,M", [([0], 1), ([0, 0, 1], 4), ([63, 64, 65], 2), ([1, 127, 128, 129, 3], 3)])
def test_attn_tiny_contexts_fewer_tiles_than_blocks(dev, ctx, M):
    """Empty and one-tile contexts on 64-key pages (the tensor-core kernel): only a few of the persistent blocks get any work, the
    others leave at once; a pair's only tile may be the one that holds this call's own rows."""
    rng = np.random.default_rng(100 + len(ctx) + M)
    c = synth.attn_case(rng, ctx, M, 64)
    o = attn_paged(bf16_dev(c["q"], dev), bf16_dev(c["k_new"], dev), bf16_dev(c["v_new"], dev), bf16_dev(c["k_pages"], dev),
                   bf16_dev(c["v_pages"], dev), i32_dev(c["block_table"], dev), i32_dev(c["ctx_len"], dev), M=M)
    _check_case(dev, c, ctx, M, 64, o)
    assert _lib.device_status() == 0


def test_attn_more_sequences_than_the_tensor_core_kernel_plans_for(dev):
    """300 sequences = 600 (sequence, KV head) pairs: beyond the 512 pairs the tcgen05 kernel plans for in shared memory, so the call
    is served by the plan kernel + mma.sync kernel with TMA tile loads; same results."""
    rng = np.random.default_rng(77)
    ctx = rng.integers(1, 200, 300)
    c = synth.attn_case(rng, ctx, 1, 64)
    o = attn_paged(bf16_dev(c["q"], dev), bf16_dev(c["k_new"], dev), bf16_dev(c["v_new"], dev), bf16_dev(c["k_pages"], dev),
                   bf16_dev(c["v_pages"], dev), i32_dev(c["block_table"], dev), i32_dev(c["ctx_len"], dev), M=1)
    sel = [0, 1, 150, 299]
    for b in sel:
        n = int(ctx[b])
        pages = c["block_table"][b]
        gather = lambda Pg: np.concatenate([Pg[p] for p in pages], axis=1)[:, :n]
        _check_rows(o[b:b + 1], c["q"][b:b + 1], c["k_new"][b:b + 1], c["v_new"][b:b + 1], gather(c["k_pages"]), gather(c["v_pages"]), 1)
    assert _lib.device_status() == 0


def test_attn_one_workspace_serves_calls_of_different_shapes(dev):
    """The arrival counters in the workspace carry an epoch tag: a workspace that starts as garbage and is reused by calls with
    different batches and contexts -- so that a pair's number of partials changes from call to call -- needs no clearing."""
    from qwen_tailor_b200._lib import check, load, ptr, stream_ptr
    lib = load()
    ws_bytes = int(lib.gqa_decode_workspace_bytes(8, 8192))
    ws = torch.randint(0, 255, (ws_bytes,), dtype=torch.uint8, device=dev)
    for seed, ctx in enumerate(([8192, 40], [300, 5000, 77, 2048, 64, 1], [4000], [8192, 40])):
        rng = np.random.default_rng(200 + seed)
        M = 4
        c = synth.attn_case(rng, ctx, M, 64)
        q, kn, vn = bf16_dev(c["q"], dev), bf16_dev(c["k_new"], dev), bf16_dev(c["v_new"], dev)
        Kd, Vd = bf16_dev(c["k_pages"], dev), bf16_dev(c["v_pages"], dev)
        bt, cl = i32_dev(c["block_table"], dev), i32_dev(c["ctx_len"], dev)
        o = torch.empty_like(q)
        check(lib.gqa_decode_paged(ptr(q), ptr(kn), ptr(vn), ptr(Kd), ptr(Vd), ptr(bt), ptr(cl), ptr(o), ptr(ws), ws_bytes, len(ctx), M, 64,
                                   bt.shape[1], Kd.shape[0], int(max(ctx)), stream_ptr(dev)), "gqa_decode_paged")
        _check_case(dev, c, ctx, M, 64, o)
    assert _lib.device_status() == 0
