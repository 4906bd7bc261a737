"""Prefix cache for hybrid recurrent / attention state, on K/V pages: stands in for the reference's ``qwen35/prefix_cache.py``.

A hybrid model cannot truncate its state to "the first p tokens": every GatedDeltaNet layer keeps one recurrent state (fp32
[16,128,128] plus a conv window [3,6144]) that is only valid at the position it was captured at.  The cache therefore holds
checkpoints: the recurrent state after ``pos`` tokens, the tokens, and the K/V rows of the full-attention layers.

Same public surface and hit rules as the reference (qwen35/prefix_cache.py:57-208) -- ``lookup`` / ``restore`` / ``insert`` /
``cat_rows`` / ``clear``, ``MIN_SPLIT`` / ``MIN_GAIN``, LRU eviction of leaves, the stats dict -- but K/V lives in a *page pool*
with the layout the paged attention kernel reads ([n_pages, 2, page_size, 256] per layer and K / V), not in per-node segments:

* a checkpoint owns a list of page numbers covering rows [0, pos).  Full pages of its parent are shared by reference count; a
  row is stored once however many checkpoints and live sequences use it (the reference stores segments [parent.pos, pos) and
  concatenates the whole chain on every restore, prefix_cache.py:134-147,171);
* ``restore_paged`` hands a live sequence the checkpoint's page numbers -- O(1) in the prefix length: only the last, partly filled
  page is copied, because the sequence will append to it; everything before is read-only for the attention kernel, which writes
  only rows at or beyond the context length;
* ``insert`` of a live paged sequence shares its full pages the same way, and copies rows only for dense ([1,2,L,256]) states;
* the recurrent state is always copied (the decode kernels update it in place), through ``gdn_state_copy`` on CUDA tensors.
``restore`` still returns the reference's dense state dict for callers that want contiguous K/V buffers.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch


def _copy_flat(dst: torch.Tensor, src: torch.Tensor, n: int, d0: int, s0: int, ny: int = 1, dstride: int = 0, sstride: int = 0):
    """dst.flat[d0 + y*dstride + i] = src.flat[s0 + y*sstride + i].  CUDA tensors go through the library's strided copy kernel;
    CPU tensors (host-logic tests only: the operators themselves have no CPU path) through torch views."""
    if n <= 0 or ny <= 0:
        return
    if dst.is_cuda:
        from .batch import blit
        blit(dst, src, n, d0, s0, ny, dstride, sstride)
        return
    df, sf = dst.view(-1), src.reshape(-1)
    for y in range(ny):
        df[d0 + y * dstride:d0 + y * dstride + n] = sf[s0 + y * sstride:s0 + y * sstride + n]


class PagePool:
    """K/V pages shared by the checkpoints and by live sequences that were restored from them.

    ``K[l]`` / ``V[l]``: [n_pages, kv_heads, page_size, head_dim] bf16 for full-attention layer l -- pass them straight to
    ``attn_paged`` with a block table made of page numbers from this pool.  Page 0 is never handed out (block tables are padded
    with it)."""

    def __init__(self, n_layers: int, n_pages: int, page_size: int = 64, kv_heads: int = 2, head_dim: int = 256, device="cuda",
                 dtype=torch.bfloat16):
        assert n_pages >= 2 and page_size > 0
        self.n_layers, self.n_pages, self.page_size, self.kv_heads, self.head_dim = n_layers, n_pages, page_size, kv_heads, head_dim
        shape = (n_pages, kv_heads, page_size, head_dim)
        self.K = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(n_layers)]
        self.V = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(n_layers)]
        self.refs = np.zeros(n_pages, np.int32)
        self.free: List[int] = list(range(n_pages - 1, 0, -1))
        self.page_bytes = 2 * n_layers * kv_heads * page_size * head_dim * self.K[0].element_size()      # one page number, all layers, K and V

    def available(self) -> int:
        return len(self.free)

    def alloc(self) -> int:
        if not self.free:
            raise MemoryError("prefix cache: the K/V page pool is exhausted")
        p = self.free.pop()
        self.refs[p] = 1
        return p

    def retain(self, pages: Sequence[int]):
        for p in pages:
            assert self.refs[p] > 0, f"page {p} is not in use"
            self.refs[p] += 1

    def release(self, pages: Sequence[int]):
        for p in pages:
            assert self.refs[p] > 0, f"page {p} released twice"
            self.refs[p] -= 1
            if self.refs[p] == 0:
                self.free.append(int(p))

    def copy_rows(self, dst_page: int, src_page: int, n_rows: int):
        """Rows [0, n_rows) of every (layer, K/V, head) of src_page -> dst_page."""
        row, per_head = self.head_dim, self.page_size * self.head_dim
        for pool in self.K + self.V:
            _copy_flat(pool, pool, n_rows * row, dst_page * self.kv_heads * per_head, src_page * self.kv_heads * per_head, ny=self.kv_heads,
                       dstride=per_head, sstride=per_head)

    def write_rows(self, page: int, row0: int, kv: Sequence, src_row0: int, n_rows: int):
        """Rows [src_row0, src_row0 + n_rows) of dense buffers kv = [(K, V)] ([1, heads, L, dim]) -> rows [row0, ...) of ``page``."""
        row, per_head = self.head_dim, self.page_size * self.head_dim
        for l, (Kd, Vd) in enumerate(kv):
            for pool, src in ((self.K[l], Kd), (self.V[l], Vd)):
                L = src.shape[2]
                _copy_flat(pool, src.contiguous(), n_rows * row, page * self.kv_heads * per_head + row0 * row, src_row0 * row, ny=self.kv_heads,
                           dstride=per_head, sstride=L * row)

    def read_rows(self, page: int, n_rows: int, kv: Sequence, dst_row0: int):
        """Rows [0, n_rows) of ``page`` -> rows [dst_row0, ...) of dense buffers kv = [(K, V)] ([1, heads, L, dim])."""
        row, per_head = self.head_dim, self.page_size * self.head_dim
        for l, (Kd, Vd) in enumerate(kv):
            for pool, dst in ((self.K[l], Kd), (self.V[l], Vd)):
                L = dst.shape[2]
                _copy_flat(dst, pool, n_rows * row, dst_row0 * row, page * self.kv_heads * per_head, ny=self.kv_heads, dstride=L * row,
                           sstride=per_head)


class Node:
    """One checkpoint.  ``pages`` covers rows [0, pos) (the leading ones are shared with the parent); ``own`` is how many of them
    this node added to the cache's footprint; ``conv`` / ``ssm``: [n_linear, 1, 3, 6144] bf16 / [n_linear, 1, 16, 128, 128] fp32."""
    __slots__ = ("parent", "pos", "toks", "pages", "own", "conv", "ssm", "last", "extra", "nbytes", "stamp", "nchild", "uid", "_pool")

    def __init__(self):
        self.parent: Optional["Node"] = None
        self.nchild = 0

    def chain(self) -> List["Node"]:
        out, n = [], self
        while n is not None:
            out.append(n)
            n = n.parent
        return out[::-1]

    @property
    def kv(self):
        """The reference's view of a node's K/V: the segment [parent.pos, pos) as one tensor [2 * n_full, 1, heads, pos - a, dim]
        (gathered from the pages; for inspection and tests -- the cache itself never concatenates)."""
        pool, a = self._pool, (self.parent.pos if self.parent is not None else 0)
        n = self.pos - a
        dev = pool.K[0].device
        bufs = [(torch.zeros((1, pool.kv_heads, n, pool.head_dim), dtype=pool.K[0].dtype, device=dev),
                 torch.zeros((1, pool.kv_heads, n, pool.head_dim), dtype=pool.K[0].dtype, device=dev)) for _ in range(pool.n_layers)]
        P = pool.page_size
        for t0 in range(a - a % P, self.pos, P):
            lo, hi = max(t0, a), min(t0 + P, self.pos)
            page = self.pages[t0 // P]
            row, per_head = pool.head_dim, P * pool.head_dim
            for l, (Kd, Vd) in enumerate(bufs):
                for src, dst in ((pool.K[l], Kd), (pool.V[l], Vd)):
                    _copy_flat(dst, src, (hi - lo) * row, (lo - a) * row, page * pool.kv_heads * per_head + (lo - t0) * row, ny=pool.kv_heads,
                               dstride=n * row, sstride=per_head)
        return torch.stack([x for k, v in bufs for x in (k, v)])


def _tensor_bytes(d) -> int:
    return sum(t.numel() * t.element_size() for t in (d or {}).values() if isinstance(t, torch.Tensor))


class PrefixCache:
    MIN_SPLIT = 32        # a shared prefix shorter than this is not worth a checkpoint of its own   (prefix_cache.py:58)
    MIN_GAIN = 32         # ... nor one that saves fewer tokens than this over the best existing hit (prefix_cache.py:59)

    def __init__(self, budget_mb=1024, enabled=True, page_size=64, kv_pages=None, kv_share=0.5):
        """budget_mb: bytes the cache may hold (recurrent states + the pages its checkpoints added).  The page pool is created at
        the first insert (it needs the layer count and the device); its capacity is ``kv_pages`` pages, or ``kv_share`` of the
        budget.  A server that runs its live sequences on the same pool (restore_paged) sizes it with ``kv_pages``, or passes its
        own ``PagePool`` (``PagedPools.pages``) as ``kv_pages``."""
        self.budget = int(budget_mb * (1 << 20))
        self.enabled = enabled
        self.page_size, self._kv_pages, self._kv_share = page_size, kv_pages, kv_share
        self.pool: Optional[PagePool] = None
        if isinstance(kv_pages, PagePool):                          # the server's own pool (PagedPools.pages): live sequences and
            self.pool, self.page_size, self._kv_pages = kv_pages, kv_pages.page_size, kv_pages.n_pages      # checkpoints share pages
        self.nodes: Dict[int, Node] = {}
        self.bytes = 0
        self._clock = 0
        self._uid = 0
        self.stats = dict(lookups=0, hits=0, hit_tokens=0, prompt_tokens=0, inserted=0, evicted=0, splits=0)
        self.last_hit = 0                      # pos of the checkpoint used by the latest lookup (0 = miss)

    # ---- small things -----------------------------------------------------------------------------
    def active(self) -> bool:
        """False bypasses the cache (the reference bypasses it in its lossy W8A8 mode, prefix_cache.py:71-78)."""
        return self.enabled

    def __len__(self):
        return len(self.nodes)

    def _touch(self, node: Optional[Node]):
        self._clock += 1
        for n in (node.chain() if node is not None else ()):
            n.stamp = self._clock

    def _ensure_pool(self, n_full: int, kv_heads: int, head_dim: int, device, dtype):
        if self.pool is None:
            per_page = 2 * n_full * kv_heads * self.page_size * head_dim * torch.empty((), dtype=dtype).element_size()
            n_pages = self._kv_pages if self._kv_pages is not None else max(2, int(self.budget * self._kv_share) // per_page + 1)
            self.pool = PagePool(n_full, n_pages, self.page_size, kv_heads, head_dim, device, dtype)
        return self.pool

    # ---- lookup -----------------------------------------------------------------------------------
    def lookup(self, ids):
        """ids: token ids of the new prompt.  Returns (node, split): the deepest checkpoint whose tokens are a prefix of ids (None =
        miss; a checkpoint that covers the whole prompt only counts if it carries ``last``), and a position (0 = none) at which the
        running prefill should drop an extra checkpoint because the prompt shares that many tokens with a stored one without
        reaching its checkpoint (prefix_cache.py:90-120)."""
        if not self.active():
            return None, 0
        prompt = np.asarray(ids, dtype=np.int32)
        S = prompt.shape[0]
        hit: Optional[Node] = None
        overlap = 0
        for nd in self.nodes.values():
            n = min(nd.pos, S)
            diff = np.flatnonzero(nd.toks[:n] != prompt[:n])
            common = n if diff.size == 0 else int(diff[0])
            if common == nd.pos:                                    # the whole checkpoint is a prefix of the prompt
                usable = nd.pos < S or nd.last is not None
                if usable and (hit is None or nd.pos > hit.pos):
                    hit = nd
            elif common < S:                                        # diverges (or the prompt ends) before the checkpoint
                overlap = max(overlap, common)
        base = hit.pos if hit is not None else 0
        split = overlap if (overlap >= self.MIN_SPLIT and overlap - base >= self.MIN_GAIN) else 0
        self.stats["lookups"] += 1
        self.stats["prompt_tokens"] += S
        self.stats["splits"] += 1 if split else 0
        self.last_hit = base
        if hit is not None:
            self.stats["hits"] += 1
            self.stats["hit_tokens"] += base
            self._touch(hit)
        return hit, split

    # ---- restore ----------------------------------------------------------------------------------
    @staticmethod
    def cat_rows(chain, get, total, axis):
        """Concatenate the per-node segments ``get(node)`` ([..., n, ...] tensors or None) along ``axis``, zero-padded to ``total``
        rows (prefix_cache.py:123-132; used by engines for per-segment extras, never for K/V here)."""
        segs = [s for s in map(get, chain) if s is not None]
        rows = sum(s.shape[axis] for s in segs)
        if rows < total:
            pad = list(segs[0].shape)
            pad[axis] = total - rows
            segs.append(segs[0].new_zeros(pad))
        return segs[0].clone() if len(segs) == 1 else torch.cat(segs, dim=axis)

    def _recurrent_copy(self, node: Node):
        conv = [torch.empty_like(node.conv[i]) for i in range(node.conv.shape[0])]
        ssm = [torch.empty_like(node.ssm[i]) for i in range(node.ssm.shape[0])]
        for i, t in enumerate(conv):
            _copy_flat(t, node.conv, t.numel(), 0, i * t.numel())
        for i, t in enumerate(ssm):
            _copy_flat(t, node.ssm, t.numel(), 0, i * t.numel())
        return conv, ssm

    def restore(self, node: Node, max_len: int):
        """The reference's dense form: ({"kv": [(K, V)] x n_full [1,2,max_len,256], "conv": [...], "ssm": [...]}, chain).  Every
        tensor is fresh -- decoding from it never touches the cached bits (tests/prefix_cache.py:161-169 of the reference).  K/V
        rows are gathered page by page."""
        assert node.pos <= max_len, (node.pos, max_len)
        pool = self.pool
        dev, dt = pool.K[0].device, pool.K[0].dtype
        kv = [(torch.zeros((1, pool.kv_heads, max_len, pool.head_dim), dtype=dt, device=dev),
               torch.zeros((1, pool.kv_heads, max_len, pool.head_dim), dtype=dt, device=dev)) for _ in range(pool.n_layers)]
        P = pool.page_size
        for i, page in enumerate(node.pages):
            pool.read_rows(page, min(P, node.pos - i * P), kv, i * P)
        conv, ssm = self._recurrent_copy(node)
        return {"kv": kv, "conv": conv, "ssm": ssm}, node.chain()

    def restore_paged(self, node: Node):
        """The paged form: ({"pages": [page numbers covering rows [0, pos)], "conv": [...], "ssm": [...]}, chain).  Full pages are
        shared with the checkpoint (reference counts); a partly filled last page is copied, because the sequence appends to it.  The
        caller owns one reference on every returned page and gives them back with ``release_pages`` (pages it allocates from
        ``self.pool`` for later tokens likewise)."""
        pool = self.pool
        P = pool.page_size
        full = node.pos // P
        pages = list(node.pages[:full])
        pool.retain(pages)
        if node.pos % P:
            self._make_room(1, protect=node)
            fresh = pool.alloc()
            pool.copy_rows(fresh, node.pages[full], node.pos % P)
            pages.append(fresh)
        conv, ssm = self._recurrent_copy(node)
        return {"pages": pages, "conv": conv, "ssm": ssm}, node.chain()

    def release_pages(self, pages: Sequence[int]):
        self.pool.release(pages)

    # ---- insert -----------------------------------------------------------------------------------
    def insert(self, parent: Optional[Node], toks, pos: int, state: dict, last=None, extra=None):
        """Checkpoint the live ``state`` (valid after ``pos`` tokens).  ``state["conv"]`` / ``["ssm"]``: per-layer tensors; K/V either
        dense, ``state["kv"]`` = [(K, V)] of [1,2,L,256] with rows [0, pos) valid (only rows from the parent's position on are read),
        or paged, ``state["pages"]`` = page numbers of ``self.pool`` covering rows [0, pos) (a sequence that came out of
        ``restore_paged`` or allocates from the pool): its full pages are shared, not copied.  ``toks``: the prompt (>= pos ids).
        ``last``: what a hit at pos == len(prompt) needs (first token ...); ``extra``: per-segment tensors of the owning engine.
        Returns the node; an existing node for identical tokens; ``parent`` when the cache is off or the node does not fit."""
        if not self.active():
            return parent
        toks = np.asarray(toks, dtype=np.int32)[:pos]
        for nd in self.nodes.values():                              # identical checkpoint: keep one
            if nd.pos == pos and np.array_equal(nd.toks, toks):
                self._touch(nd)
                if nd.last is None and last is not None:
                    nd.last = {k: (v.clone() if isinstance(v, torch.Tensor) else v) for k, v in last.items()}
                    nd.nbytes += _tensor_bytes(nd.last)
                    self.bytes += _tensor_bytes(nd.last)
                return nd
        a = parent.pos if parent is not None else 0
        assert pos > a, (pos, a)
        conv0, ssm0 = state["conv"][0], state["ssm"][0]
        paged = "pages" in state
        if paged:
            assert self.pool is not None, "a paged state must live in this cache's pool"
            pool = self.pool
        else:
            K0 = state["kv"][0][0]
            pool = self._ensure_pool(len(state["kv"]), K0.shape[1], K0.shape[3], K0.device, K0.dtype)
        P = pool.page_size
        n_total = (pos + P - 1) // P
        shared = a // P if parent is not None else 0               # full pages of the parent
        fixed = (sum(t.numel() * t.element_size() for t in state["conv"]) + sum(t.numel() * t.element_size() for t in state["ssm"])
                 + _tensor_bytes(last) + _tensor_bytes(extra))
        nbytes = fixed + (n_total - shared) * pool.page_bytes
        if nbytes > self.budget:
            return parent                                           # an oversize node is not stored (prefix_cache.py:175-176)
        need = (n_total - shared) if not paged else (1 if pos % P else 0)
        if not self._make_room(need, protect=parent):
            return parent

        nd = Node()
        nd._pool, nd.parent, nd.pos, nd.toks = pool, parent, pos, toks.copy()
        pages = list(parent.pages[:shared]) if parent is not None else []
        pool.retain(pages)
        if paged:
            src = list(state["pages"])
            assert len(src) >= n_total, "state['pages'] does not cover rows [0, pos)"
            full = pos // P
            pool.retain(src[shared:full])                           # shared with the live sequence: zero copies
            pages += src[shared:full]
            if pos % P:                                             # the sequence keeps appending to its last page: take a copy
                fresh = pool.alloc()
                pool.copy_rows(fresh, src[full], pos % P)
                pages.append(fresh)
        else:
            for i in range(shared, n_total):
                page = pool.alloc()
                lo = i * P
                if lo < a:                                          # the parent's partly filled page: its rows first, then ours
                    pool.copy_rows(page, parent.pages[i], a - lo)
                    lo = a
                pool.write_rows(page, lo - i * P, state["kv"], lo, min((i + 1) * P, pos) - lo)
                pages.append(page)
        nd.pages, nd.own = pages, n_total - shared
        nd.conv = torch.empty((len(state["conv"]),) + tuple(conv0.shape), dtype=conv0.dtype, device=conv0.device)
        nd.ssm = torch.empty((len(state["ssm"]),) + tuple(ssm0.shape), dtype=ssm0.dtype, device=ssm0.device)
        for i, t in enumerate(state["conv"]):
            _copy_flat(nd.conv, t.contiguous(), t.numel(), i * t.numel(), 0)
        for i, t in enumerate(state["ssm"]):
            _copy_flat(nd.ssm, t.contiguous(), t.numel(), i * t.numel(), 0)
        nd.last = None if last is None else {k: (v.clone() if isinstance(v, torch.Tensor) else v) for k, v in last.items()}
        nd.extra = extra
        nd.nbytes = nbytes
        self._uid += 1
        nd.uid = self._uid
        self.nodes[nd.uid] = nd
        if parent is not None:
            parent.nchild += 1
        self.bytes += nbytes
        self.stats["inserted"] += 1
        self._touch(nd)
        self._evict(protect=nd)
        return nd

    # ---- eviction ---------------------------------------------------------------------------------
    def _drop(self, node: Node):
        del self.nodes[node.uid]
        if node.parent is not None:
            node.parent.nchild -= 1
        self.pool.release(node.pages)
        self.bytes -= node.nbytes
        self.stats["evicted"] += 1

    def _victim(self, protect: Optional[Node]) -> Optional[Node]:
        """Least recently used leaf outside the chain that is being built or used (prefix_cache.py:189-204)."""
        keep = {n.uid for n in protect.chain()} if protect is not None and hasattr(protect, "uid") else set()
        leaves = [n for n in self.nodes.values() if n.nchild == 0 and n.uid not in keep]
        return min(leaves, key=lambda n: n.stamp) if leaves else None

    def _evict(self, protect: Optional[Node] = None):
        while self.bytes > self.budget:
            v = self._victim(protect)
            if v is None:
                break
            self._drop(v)

    def _make_room(self, n_pages: int, protect: Optional[Node] = None) -> bool:
        """Free pages by evicting leaves until ``n_pages`` can be allocated; False if that is impossible."""
        if self.pool is not None and n_pages > self.pool.n_pages - 1:
            return False                                            # more than the pool holds: evicting would not help
        while self.pool is not None and self.pool.available() < n_pages:
            v = self._victim(protect)
            if v is None:
                return False
            self._drop(v)
        return True

    def clear(self):
        for n in list(self.nodes.values()):
            self.pool.release(n.pages)
        self.nodes.clear()
        self.bytes = 0
