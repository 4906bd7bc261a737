"""Sharding of the hot path over the GPUs of one node (one process per GPU, ``torch.distributed``).

The reference is single-GPU; nothing here has a counterpart in it.  Two partitions exist:

* by sequence -- decode, speculative verify and ragged prefill batches: sequences (and their slots, pages and snapshot
  entries) are independent, so ranks work on disjoint sequences and nothing is exchanged on the data path;
* by head group -- prefill of one long sequence: the 16 heads of the gated delta rule are independent, rank r computes heads
  [16 r / n, 16 (r + 1) / n) with its slice of the fp32 state staying resident, and the only exchange is one all-gather of the
  bf16 outputs (T x 2048 x 2 bytes in total per layer).
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist


def partition_sequences(lengths: Sequence[int], n_ranks: int) -> List[List[int]]:
    """Greedy longest-first assignment of sequences to ranks by token count (ragged batches: balances the work, not the count).
    Returns, per rank, the sorted indices of its sequences; every sequence appears exactly once."""
    order = sorted(range(len(lengths)), key=lambda i: (-int(lengths[i]), i))
    loads = [0] * n_ranks
    parts: List[List[int]] = [[] for _ in range(n_ranks)]
    for i in order:
        r = min(range(n_ranks), key=lambda j: (loads[j], j))
        parts[r].append(i)
        loads[r] += int(lengths[i])
    return [sorted(p) for p in parts]


def head_range(rank: int, world: int, n_heads: int = 16) -> Tuple[int, int]:
    """Heads [lo, hi) owned by ``rank`` when ``n_heads`` are split evenly over ``world`` ranks."""
    if n_heads % world:
        raise ValueError(f"{n_heads} heads cannot be split evenly over {world} ranks")
    per = n_heads // world
    return rank * per, (rank + 1) * per


def gather_heads(y: torch.Tensor, rank: int, world: int, group=None) -> torch.Tensor:
    """All-gather head-sharded outputs.  ``y`` is [T, H, D] with this rank's heads ``head_range(rank, world, H)`` filled in;
    on return every rank's slice is filled in (in place; returns ``y``).  One collective of T*H*D elements in total."""
    if world == 1:
        return y
    T, H, D = y.shape
    lo, hi = head_range(rank, world, H)
    mine = y[:, lo:hi, :].contiguous()
    out = torch.empty((world, T, hi - lo, D), dtype=y.dtype, device=y.device)
    dist.all_gather_into_tensor(out.view(world * T, hi - lo, D), mine, group=group)
    y.copy_(out.permute(1, 0, 2, 3).reshape(T, H, D))
    return y


def prefill_head_sharded(q, k, v, lg, beta, cu_seqlens, rank: int, world: int, init_state=None, init_idx=None, group=None):
    """Chunked prefill of a packed batch with the heads split over ``world`` ranks.  Every rank holds the full q/k/v/lg/beta
    (they are inputs of the layer) but computes only its heads; y is all-gathered, the final states stay sharded:
    returns (y [T, H, 128] complete on every rank, final_state [n_seq, H, 128, 128] valid for heads head_range(rank, world))."""
    from .gdn_nax import gdn_chunked_varlen
    lo, hi = head_range(rank, world, q.shape[1])
    y, st = gdn_chunked_varlen(q, k, v, lg, beta, cu_seqlens, init_state=init_state, init_idx=init_idx, head_lo=lo, head_hi=hi)
    gather_heads(y, rank, world, group)
    return y, st


def shard_varlen_batch(lengths: Sequence[int], rank: int, world: int):
    """Sequence-sharding of a packed ragged batch: returns (indices of this rank's sequences, their token ranges in the packed
    global layout as (start, end) pairs, local cu_seqlens as a list)."""
    parts = partition_sequences(lengths, world)
    starts = [0]
    for n in lengths:
        starts.append(starts[-1] + int(n))
    mine = parts[rank]
    ranges = [(starts[i], starts[i + 1]) for i in mine]
    cu = [0]
    for a, b in ranges:
        cu.append(cu[-1] + (b - a))
    return mine, ranges, cu


def bind_host_to_gpu(device_index: int) -> dict:
    """Pin the calling process to the CPUs of the NUMA node the GPU hangs off, so that pinned host buffers allocated afterwards lie
    in that node's memory and host<->device copies do not cross the socket interconnect.  With eight ranks each moving tens of GB/s
    between pinned memory and its GPU, copies through the other socket's memory are what saturates first.  Changes nothing on the
    GPU; a no-op (reported in the returned dict) where the platform does not expose the topology.  Linux only."""
    import os
    info = {"bound": False}
    try:
        p = torch.cuda.get_device_properties(device_index)
        bdf = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
        info.update(pci=bdf, numa_node=node)
        if node < 0:
            return info
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            spec = f.read().strip()
        cpus = set()
        for part in spec.split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return info
        os.sched_setaffinity(0, allowed)
        info.update(bound=True, cpus=len(allowed))
    except (OSError, ValueError, AttributeError, RuntimeError) as e:
        info["error"] = type(e).__name__
    return info
