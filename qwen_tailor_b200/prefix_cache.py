"""Prefix cache for hybrid recurrent/attention state: drop-in for the reference's ``qwen35/prefix_cache.py``.

A hybrid model cannot truncate its state to "the first p tokens": every GatedDeltaNet layer keeps one recurrent state (fp32
[1,16,128,128] plus a conv window [1,3,6144]) that is only valid at the position it was captured at.  The cache therefore
holds checkpoints (nodes): the complete recurrent state after ``pos`` tokens, the tokens themselves, and the K/V rows
``[parent.pos, pos)`` of the full-attention layers as a segment, so a chain of checkpoints of one prompt stores each K/V row
once.  ``lookup`` finds the deepest checkpoint that is a prefix of a new prompt (longest common prefix over the stored token
arrays) and proposes a split position when the prompt only partly overlaps a stored one; ``restore`` rebuilds a live state;
``insert`` checkpoints a live state; eviction removes the least recently used leaf until the byte budget holds.
(Behaviour of qwen35/prefix_cache.py:57-208.)

Difference forced by mutable tensors: the reference shares the recurrent arrays of a node with the restored state because MLX
arrays are immutable values; here the decode kernels update state in place, so ``restore`` hands out copies and ``insert``
stores copies -- a restored state can be decoded from without touching the cached bits.  All copies are device-to-device.
"""
from __future__ import annotations

import numpy as np
import torch


class Node:
    __slots__ = ("parent", "pos", "toks", "kv", "conv", "ssm", "last", "extra", "nbytes", "stamp", "nchild", "uid")

    def __init__(self):
        self.parent = None
        self.nchild = 0

    def chain(self):
        out, n = [], self
        while n is not None:
            out.append(n)
            n = n.parent
        out.reverse()
        return out


def _nb(*items):
    return sum(t.numel() * t.element_size() for t in items if isinstance(t, torch.Tensor))


def _own(d):
    """Copy the tensors of dict ``d`` into storage of their own (a view would keep a whole activation alive)."""
    return None if d is None else {k: (v.clone() if isinstance(v, torch.Tensor) else v) for k, v in d.items()}


class PrefixCache:
    MIN_SPLIT = 32        # a shared prefix shorter than this is not worth a checkpoint of its own
    MIN_GAIN = 32         # ... nor one that saves fewer tokens than this over the best existing hit

    def __init__(self, budget_mb=1024, enabled=True):
        self.budget = int(budget_mb * (1 << 20))
        self.enabled = enabled
        self.nodes: dict[int, Node] = {}
        self.bytes = 0
        self._clock = 0
        self._uid = 0
        self.stats = dict(lookups=0, hits=0, hit_tokens=0, prompt_tokens=0, inserted=0, evicted=0, splits=0)
        self.last_hit = 0                      # pos of the checkpoint used by the latest lookup (0 = miss)

    # ---- helpers ----------------------------------------------------------------------------------
    def active(self):
        """False bypasses the cache (the reference bypasses it in its lossy W8A8 mode, prefix_cache.py:71-78)."""
        return self.enabled

    def _touch(self, node):
        self._clock += 1
        while node is not None:
            node.stamp = self._clock
            node = node.parent

    def __len__(self):
        return len(self.nodes)

    # ---- lookup -----------------------------------------------------------------------------------
    def lookup(self, ids):
        """ids: token ids of the new prompt.  Returns (node, split): the deepest checkpoint that is a prefix of ids (None = miss; a
        checkpoint covering the whole prompt only counts if it carries the first token), and a position (0 = none) at which the new
        prefill should add a checkpoint because the prompt overlaps a stored one up to there."""
        if not self.active():
            return None, 0
        t = np.asarray(ids, dtype=np.int32)
        S = len(t)
        best, part = None, 0
        for nd in self.nodes.values():
            n = min(nd.pos, S)
            eq = nd.toks[:n] == t[:n]
            lcp = n if eq.all() else int(eq.argmin())
            if lcp == nd.pos:
                if (nd.pos < S or nd.last is not None) and (best is None or nd.pos > best.pos):
                    best = nd
            elif lcp < S:
                part = max(part, lcp)
        base = best.pos if best is not None else 0
        split = part if (part >= self.MIN_SPLIT and part - base >= self.MIN_GAIN) else 0
        st = self.stats
        st["lookups"] += 1
        st["prompt_tokens"] += S
        self.last_hit = base
        if best is not None:
            st["hits"] += 1
            st["hit_tokens"] += base
            self._touch(best)
        if split:
            st["splits"] += 1
        return best, split

    # ---- restore ----------------------------------------------------------------------------------
    @staticmethod
    def cat_rows(chain, get, total, axis):
        """Concatenate the per-node segments ``get(node)`` ([..., n, ...] tensors or None) along ``axis``, zero-padded to ``total`` rows."""
        parts = [g for g in (get(c) for c in chain) if g is not None]
        have = sum(p.shape[axis] for p in parts)
        if total > have:
            shp = list(parts[0].shape)
            shp[axis] = total - have
            parts.append(torch.zeros(shp, dtype=parts[0].dtype, device=parts[0].device))
        return torch.cat(parts, dim=axis) if len(parts) > 1 else parts[0].clone()

    def restore(self, node, max_len):
        """State dict of the checkpoint ({"kv": [(K, V)] x n_full [1,2,max_len,256], "conv": [...], "ssm": [...]}) and its chain.
        Every tensor is fresh: K/V are the chain's segments concatenated and zero-padded, the recurrent tensors are copies."""
        assert node.pos <= max_len, (node.pos, max_len)
        chain = node.chain()
        nb = node.kv.shape[0]
        bufs = []
        for j in range(nb):
            parts = [c.kv[j] for c in chain]
            if max_len > node.pos:
                parts.append(torch.zeros((1, node.kv.shape[2], max_len - node.pos, node.kv.shape[4]), dtype=node.kv.dtype, device=node.kv.device))
            bufs.append(torch.cat(parts, dim=2) if len(parts) > 1 else parts[0].clone())
        st = {"kv": [(bufs[2 * i], bufs[2 * i + 1]) for i in range(nb // 2)],
              "conv": [node.conv[i].clone() for i in range(node.conv.shape[0])], "ssm": [node.ssm[i].clone() for i in range(node.ssm.shape[0])]}
        return st, chain

    # ---- insert -----------------------------------------------------------------------------------
    def insert(self, parent, toks, pos, state, last=None, extra=None):
        """Checkpoint the live ``state`` (valid after ``pos`` tokens, K/V rows [parent.pos : pos) are the new ones).  ``toks``: the
        prompt's token ids (>= pos long).  ``last``: optional dict with what a hit at pos == len(prompt) needs (first token ...);
        ``extra``: dict of per-segment tensors for the owning engine.  Returns the node (an existing one for identical tokens)."""
        if not self.active():
            return parent
        toks = np.asarray(toks, dtype=np.int32)
        for nd in self.nodes.values():
            if nd.pos == pos and np.array_equal(nd.toks, toks[:pos]):
                self._touch(nd)
                if nd.last is None and last is not None:
                    nd.last = _own(last)
                    nd.nbytes += _nb(*nd.last.values())
                    self.bytes += _nb(*nd.last.values())
                return nd
        a = parent.pos if parent is not None else 0
        assert pos > a
        nd = Node()
        nd.parent, nd.pos, nd.toks = parent, pos, toks[:pos].copy()
        nd.kv = torch.stack([x[:, :, a:pos] for k, v in state["kv"] for x in (k, v)])      # [2*n_full, 1, 2, pos-a, 256], a real copy
        nd.conv, nd.ssm = torch.stack(list(state["conv"])), torch.stack(list(state["ssm"]))  # real copies
        nd.last, nd.extra = _own(last), extra
        nd.nbytes = _nb(nd.kv, nd.conv, nd.ssm) + _nb(*(nd.last or {}).values()) + _nb(*(extra or {}).values())
        if nd.nbytes > self.budget:
            return parent
        self._uid += 1
        nd.uid = self._uid
        self.nodes[nd.uid] = nd
        if parent is not None:
            parent.nchild += 1
        self.bytes += nd.nbytes
        self.stats["inserted"] += 1
        self._touch(nd)
        self._evict(protect=nd)
        return nd

    def _evict(self, protect=None):
        keep = set()
        n = protect
        while n is not None:                    # the chain being built / used stays
            keep.add(n.uid)
            n = n.parent
        while self.bytes > self.budget:
            leaves = [n for n in self.nodes.values() if n.nchild == 0 and n.uid not in keep]
            if not leaves:
                break
            v = min(leaves, key=lambda n: n.stamp)
            del self.nodes[v.uid]
            if v.parent is not None:
                v.parent.nchild -= 1
            self.bytes -= v.nbytes
            self.stats["evicted"] += 1

    def clear(self):
        self.nodes.clear()
        self.bytes = 0
