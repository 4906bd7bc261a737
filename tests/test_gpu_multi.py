"""Two-GPU test of the head-group sharding of one long prefill (NCCL all-gather of the outputs) and of sequence sharding.
Skipped unless two CUDA devices are visible."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from qwen_tailor_b200 import synth
        from qwen_tailor_b200.gated_delta import gates
        from qwen_tailor_b200.gdn_nax import gdn_chunked_varlen
        from qwen_tailor_b200.shard import head_range, prefill_head_sharded, shard_varlen_batch
        T = 700
        c = synth.config3_layer(3, T)
        tb = lambda x: torch.from_numpy(np.ascontiguousarray(x, np.float32)).to(dev).to(torch.bfloat16)
        tf = lambda x: torch.from_numpy(np.ascontiguousarray(x, np.float32)).to(dev)
        q, k, v = tb(c["q"]), tb(c["k"]), tb(c["v"])
        _, lg, beta = gates(tb(c["a"]), tb(c["b"]), tf(c["A_log"]), tf(c["dt_bias"]))
        cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
        y_full, s_full = gdn_chunked_varlen(q, k, v, lg, beta, cu)                       # every rank: the unsharded result
        y, s = prefill_head_sharded(q, k, v, lg, beta, cu, rank, world)
        lo, hi = head_range(rank, world)
        assert torch.equal(y, y_full), "all-gathered outputs must equal the single-GPU result bit for bit"
        assert torch.equal(s[:, lo:hi], s_full[:, lo:hi])
        # sequence sharding of a ragged batch: each rank runs its own sequences, no collective on the data path
        lengths = [130, 64, 257, 5]
        mine, ranges, cu_l = shard_varlen_batch(lengths, rank, world)
        tot = sum(lengths)
        c4 = synth.config3_layer(4, tot)
        q4, k4, v4 = tb(c4["q"]), tb(c4["k"]), tb(c4["v"])
        _, lg4, b4 = gates(tb(c4["a"]), tb(c4["b"]), tf(c4["A_log"]), tf(c4["dt_bias"]))
        cu_g = torch.tensor(np.concatenate([[0], np.cumsum(lengths)]), dtype=torch.int32, device=dev)
        yg, sg = gdn_chunked_varlen(q4, k4, v4, lg4, b4, cu_g)
        sel = torch.cat([torch.arange(a, b, device=dev) for a, b in ranges])
        yl, sl = gdn_chunked_varlen(q4[sel].contiguous(), k4[sel].contiguous(), v4[sel].contiguous(), lg4[sel].contiguous(), b4[sel].contiguous(),
                                    torch.tensor(cu_l, dtype=torch.int32, device=dev))
        assert torch.equal(yl, yg[sel]) and torch.equal(sl, sg[mine])
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_head_and_sequence_sharding_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mp.spawn(_worker, args=(2, _free_port()), nprocs=2, join=True)
