"""CPU tests of the host-side logic: prefix cache (behaviour of the reference's tests/prefix_cache.py that does not need a model),
sequence / head sharding, and the world-size-2 gloo path of the head all-gather."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from qwen_tailor_b200.prefix_cache import PrefixCache
from qwen_tailor_b200.shard import gather_heads, head_range, partition_sequences, shard_varlen_batch


def _state(pos, max_len, seed, n_lin=3, n_full=2):
    g = torch.Generator().manual_seed(seed)
    kv = []
    for _ in range(n_full):
        K = torch.zeros((1, 2, max_len, 256), dtype=torch.bfloat16)
        V = torch.zeros((1, 2, max_len, 256), dtype=torch.bfloat16)
        K[:, :, :pos] = torch.randn((1, 2, pos, 256), generator=g).to(torch.bfloat16)
        V[:, :, :pos] = torch.randn((1, 2, pos, 256), generator=g).to(torch.bfloat16)
        kv.append((K, V))
    return {"kv": kv, "conv": [torch.randn((1, 3, 6144), generator=g).to(torch.bfloat16) for _ in range(n_lin)],
            "ssm": [torch.randn((1, 16, 128, 128), generator=g) for _ in range(n_lin)]}


def _extend(st, a, pos, seed):
    """A later state of the same sequence: K/V rows [a, pos) appended, recurrent state replaced."""
    new = _state(pos, st["kv"][0][0].shape[2], seed, len(st["conv"]), len(st["kv"]))
    for (K, V), (K0, V0) in zip(new["kv"], st["kv"]):
        K[:, :, :a] = K0[:, :, :a]
        V[:, :, :a] = V0[:, :, :a]
    return new


def test_prefix_cache_hit_restore_and_aliasing():
    pc = PrefixCache(budget_mb=64)
    toks = np.arange(1000, 1300, dtype=np.int32)
    st100 = _state(100, 256, 1)
    n1 = pc.insert(None, toks, 100, st100)
    st200 = _extend(st100, 100, 200, 2)
    n2 = pc.insert(n1, toks, 200, st200, last={"h": torch.ones(1, 8)})
    assert n2.kv.shape[3] == 100, "K/V rows are stored once per token: the child holds only rows [100, 200)"
    # deepest prefix wins; a checkpoint that covers the whole prompt only counts if it carries `last`
    node, split = pc.lookup(toks[:250])
    assert node is n2 and split == 0 and pc.last_hit == 200
    node, _ = pc.lookup(toks[:200])
    assert node is n2
    node, _ = pc.lookup(toks[:100])
    assert node is None, "n1 covers the whole prompt but has no `last`"
    node, _ = pc.lookup(toks[:150])
    assert node is n1
    st, chain = pc.restore(n2, 256)
    assert [c.pos for c in chain] == [100, 200]
    for (K, V), (K0, V0) in zip(st["kv"], st200["kv"]):
        assert torch.equal(K, K0) and torch.equal(V, V0)
    assert all(torch.equal(a, b) for a, b in zip(st["ssm"], st200["ssm"])) and all(torch.equal(a, b) for a, b in zip(st["conv"], st200["conv"]))
    # decoding from a restored state (in-place updates) must leave the cached bits unchanged
    before = n2.ssm.clone()
    for s in st["ssm"]:
        s.mul_(0).add_(7)
    st["kv"][0][0].fill_(3)
    assert torch.equal(n2.ssm, before)
    st_again, _ = pc.restore(n2, 256)
    assert all(torch.equal(a, b) for a, b in zip(st_again["ssm"], st200["ssm"]))
    # the live state that was checkpointed can be mutated too
    st200["ssm"][0].zero_()
    assert torch.equal(n2.ssm, before)
    assert pc.stats["hits"] == 3 and pc.stats["inserted"] == 2


def test_prefix_cache_pages_are_shared_not_copied():
    """K/V lives in pages: a child shares its parent's full pages, a paged restore shares the checkpoint's full pages and copies
    only the partly filled last one, and a live paged sequence is checkpointed without copying its full pages."""
    pc = PrefixCache(budget_mb=64, page_size=64, kv_pages=64)
    toks = np.arange(3000, 3400, dtype=np.int32)
    st = _state(300, 320, 5)
    n1 = pc.insert(None, toks, 160, st)                               # pages 0, 1 full, page 2 holds rows 128..159
    pool = pc.pool
    assert len(n1.pages) == 3 and n1.own == 3 and pool.available() == 63 - 3
    n2 = pc.insert(n1, toks, 300, st)                                 # shares pages 0, 1; own pages for rows 128..299
    assert n2.pages[:2] == n1.pages[:2] and n2.pages[2] != n1.pages[2] and len(n2.pages) == 5 and n2.own == 3
    assert list(pool.refs[n1.pages[:2]]) == [2, 2] and pool.refs[n1.pages[2]] == 1
    assert n2.kv.shape[3] == 140                                      # the reference's segment view: rows [160, 300)
    dense, _ = pc.restore(n2, 320)
    for (K, V), (K0, V0) in zip(dense["kv"], st["kv"]):
        assert torch.equal(K[:, :, :300], K0[:, :, :300]) and torch.equal(V[:, :, :300], V0[:, :, :300]) and float(K[:, :, 300:].abs().max()) == 0
    # paged restore: full pages by reference, the partial page by copy
    live, chain = pc.restore_paged(n2)
    assert [c.pos for c in chain] == [160, 300]
    assert live["pages"][:4] == n2.pages[:4] and live["pages"][4] != n2.pages[4]
    assert list(pool.refs[n2.pages[:2]]) == [3, 3] and pool.refs[live["pages"][4]] == 1
    tail = live["pages"][4]
    assert torch.equal(pool.K[0][tail, :, :300 - 256], pool.K[0][n2.pages[4], :, :300 - 256])
    # the live sequence appends rows 300..319 to its own copy of the last page; the checkpoint's page is untouched
    before = pool.K[0][n2.pages[4]].clone()
    pool.K[0][tail, :, 300 - 256:] = 7
    assert torch.equal(pool.K[0][n2.pages[4]], before)
    # checkpoint the live sequence at 320 (page-aligned): nothing is copied, its five pages are shared
    free_before = pool.available()
    n3 = pc.insert(n2, np.concatenate([toks[:300], np.arange(20, dtype=np.int32)]), 320, {"pages": live["pages"], "conv": live["conv"], "ssm": live["ssm"]})
    assert n3.pages == live["pages"] and pool.available() == free_before and pool.refs[tail] == 2 and n3.own == 1
    pc.release_pages(live["pages"])
    assert pool.refs[tail] == 1 and list(pool.refs[n1.pages[:2]]) == [3, 3]          # n1, n2, n3
    pc.clear()
    assert pool.available() == 63 and int(pool.refs.sum()) == 0


def test_prefix_cache_page_pool_exhaustion_evicts_leaves():
    pc = PrefixCache(budget_mb=512, page_size=64, kv_pages=7)          # 6 usable pages
    a = pc.insert(None, np.arange(0, 200, dtype=np.int32), 192, _state(192, 256, 1))       # 3 pages
    b = pc.insert(None, np.arange(1000, 1200, dtype=np.int32), 192, _state(192, 256, 2))   # 3 pages: pool full
    assert pc.pool.available() == 0
    c = pc.insert(None, np.arange(2000, 2200, dtype=np.int32), 128, _state(128, 256, 3))   # needs 2: the LRU leaf (a) goes
    assert c is not None and a.uid not in pc.nodes and b.uid in pc.nodes and pc.stats["evicted"] == 1
    assert pc.insert(None, np.arange(5000, 5600, dtype=np.int32), 512, _state(512, 512, 4)) is None, "8 pages can never fit"


def test_prefix_cache_split_learning_and_identical_insert():
    pc = PrefixCache(budget_mb=64)
    a = np.arange(0, 200, dtype=np.int32)
    pc.insert(None, a, 200, _state(200, 256, 1))
    b = np.concatenate([a[:120], np.arange(5000, 5100, dtype=np.int32)])
    node, split = pc.lookup(b)
    assert node is None and split == 120, "a partial overlap of 120 >= MIN_SPLIT tokens proposes a checkpoint there"
    node, split = pc.lookup(np.concatenate([a[:20], b[120:]]))
    assert node is None and split == 0
    n = pc.insert(None, b, 120, _state(120, 256, 3))
    assert pc.insert(None, b, 120, _state(120, 256, 4)) is n, "identical tokens return the existing node"
    node, split = pc.lookup(b)
    assert node is n and split == 0


def test_prefix_cache_lru_eviction_and_budget():
    one = 3 * (16 * 128 * 128 * 4 + 3 * 6144 * 2) + 4 * 2 * 64 * 256 * 2
    pc = PrefixCache(budget_mb=2.5 * one / (1 << 20))
    nodes = []
    for i in range(3):
        t = np.arange(i * 1000, i * 1000 + 64, dtype=np.int32)
        nodes.append(pc.insert(None, t, 64, _state(64, 128, i)))
    assert len(pc) == 2 and pc.stats["evicted"] == 1 and nodes[0].uid not in pc.nodes, "least recently used leaf goes first"
    pc.lookup(np.arange(1000, 1100, dtype=np.int32))                      # touch node 1
    pc.insert(None, np.arange(9000, 9064, dtype=np.int32), 64, _state(64, 128, 9))
    assert nodes[1].uid in pc.nodes and nodes[2].uid not in pc.nodes
    big = PrefixCache(budget_mb=0.5)
    assert big.insert(None, np.arange(64, dtype=np.int32), 64, _state(64, 128, 0)) is None and len(big) == 0, "oversize node not stored"
    off = PrefixCache(enabled=False)
    assert off.lookup([1, 2, 3]) == (None, 0) and off.insert(None, [1, 2, 3], 3, _state(3, 8, 0)) is None
    pc.clear()
    assert len(pc) == 0 and pc.bytes == 0


def test_cat_rows_pads_with_zeros():
    class C:
        def __init__(self, seg):
            self.seg = seg
    a, b = torch.ones((1, 2, 3, 4)), 2 * torch.ones((1, 2, 5, 4))
    out = PrefixCache.cat_rows([C(a), C(None), C(b)], lambda c: c.seg, 10, 2)
    assert out.shape == (1, 2, 10, 4) and float(out[:, :, :3].min()) == 1 and float(out[:, :, 3:8].min()) == 2 and float(out[:, :, 8:].abs().max()) == 0


def test_partition_sequences_balances_tokens():
    rng = np.random.default_rng(7)
    lengths = rng.integers(128, 4097, 16)
    for world in (1, 2, 4, 8):
        parts = partition_sequences(lengths, world)
        assert sorted(i for p in parts for i in p) == list(range(16))
        loads = [int(sum(lengths[i] for i in p)) for p in parts]
        assert max(loads) - min(loads) <= int(lengths.max())
    mine, ranges, cu = shard_varlen_batch([5, 0, 7, 3], 1, 2)
    assert len(mine) == len(ranges) == len(cu) - 1 and cu[-1] == sum(b - a for a, b in ranges)
    assert head_range(3, 8) == (6, 8) and head_range(0, 1) == (0, 16)
    with pytest.raises(ValueError):
        head_range(0, 3)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gather_worker(rank, world, port, T):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        want = torch.arange(T * 16 * 8, dtype=torch.float32).reshape(T, 16, 8).to(torch.bfloat16)
        y = torch.full_like(want, -1.0)
        lo, hi = head_range(rank, world)
        y[:, lo:hi] = want[:, lo:hi]                       # what the head-sharded kernel call leaves behind on this rank
        gather_heads(y, rank, world)
        assert torch.equal(y, want)
        # sequence sharding needs no collective: the union of the ranks' sequences is the batch
        lengths = [300, 64, 1000, 129, 5, 77]
        mine, _, _ = shard_varlen_batch(lengths, rank, world)
        got = [None] * world
        dist.all_gather_object(got, mine)
        assert sorted(i for p in got for i in p) == list(range(len(lengths)))
    finally:
        dist.destroy_process_group()


def test_gather_heads_world_size_2_gloo():
    mp.spawn(_gather_worker, args=(2, _free_port(), 37), nprocs=2, join=True)


def test_bind_host_to_gpu_is_harmless_without_a_gpu():
    """The NUMA binding used by the multi-GPU bench reports what it did and never raises, whatever the platform exposes."""
    from qwen_tailor_b200.shard import bind_host_to_gpu
    before = os.sched_getaffinity(0)
    info = bind_host_to_gpu(0)
    assert isinstance(info, dict) and "bound" in info
    if not info["bound"]:
        assert os.sched_getaffinity(0) == before


def test_workspace_sizing_functions_need_no_gpu():
    """Host arithmetic of the C ABI: the record buffer of a packed prefill batch and the prefill-attention workspace."""
    from qwen_tailor_b200 import _lib
    lib = _lib.load()
    # one record of 17,152 bytes per (chunk, head); a sequence of T tokens owns T // 64 + 1 chunk slots
    assert lib.gdn_prefill_workspace_bytes(1, 2048, 16) == (2048 // 64 + 1) * 16 * 17152
    assert lib.gdn_prefill_workspace_bytes(3, 64 + 1 + 130, 16) == ((64 + 1 + 130) // 64 + 3) * 16 * 17152
    assert lib.gqa_prefill_attn_workspace_bytes(1024, 0) > 0          # short prefill: the heaviest query blocks may be split
    assert lib.gqa_prefill_attn_workspace_bytes(4096, 0) == 0         # long prefill: more than one block per SM already
    assert lib.gqa_prefill_attn_workspace_bytes(64, 0) == 0           # a single tile per block: nothing to split
    assert lib.gqa_decode_workspace_bytes(16, 8192) > 16 * 2 * 16 * 256 * 4
