"""Slot pools of the batched decode step with the K/V cache in shared pages.

The reference keeps one contiguous K/V region per slot (``Pools``, qwen35/batch.py:405-462: [S+1, 2, Lmax, 256]) and copies K/V on
every admission and every prefix-cache hit (qwen35/serve.py:297-308, prefix_cache.py:134-147).  Here the recurrent state lives in
slot pools as before, but K/V lives in the ``PagePool`` that the prefix cache also uses: a slot is a row of the block table, a
prefix-cache hit hands the slot the checkpoint's page numbers (no K/V copy), and pages are allocated as the sequence grows.
The attention kernel reads the pool and the table directly (``attn``).  Nothing here has a line-by-line counterpart in the reference.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from .batch import CD, DK, DV, HV, attn_paged, blit, deltanet_b
from .config import Cfg
from .prefix_cache import PagePool


class PagedPools:
    """``slots`` sequences: conv / ssm slot pools for the GatedDeltaNet layers (slot ``slots`` is the trash slot, as in ``Pools``)
    and one block-table row per slot into ``pages`` (K/V of the full-attention layers)."""

    def __init__(self, cfg: Cfg, slots: int, max_len: int, pages: Optional[PagePool] = None, n_pages: Optional[int] = None,
                 page_size: int = 64, device="cuda"):
        self.cfg, self.S, self.Lmax = cfg, slots, max_len
        self.max_pages = (max_len + page_size - 1) // page_size
        if pages is None:
            pages = PagePool(cfg.n_full, n_pages or slots * self.max_pages + 1, page_size, cfg.n_kv, cfg.head_dim, device=device)
        assert pages.page_size == page_size and pages.n_layers == cfg.n_full
        self.pages = pages
        self.conv = [torch.zeros(((slots + 1) * 2, 3, CD), dtype=torch.bfloat16, device=device) for _ in range(cfg.n_linear)]
        self.ssm = [torch.zeros((slots + 1, HV, DV, DK), dtype=torch.float32, device=device) for _ in range(cfg.n_linear)]
        self.table_host = np.zeros((slots + 1, self.max_pages), np.int32)     # page 0 pads
        self.table = torch.zeros((slots + 1, self.max_pages), dtype=torch.int32, device=device)
        self.owned: List[List[int]] = [[] for _ in range(slots + 1)]          # pages each slot holds a reference on, in order
        self.length = np.zeros(slots + 1, np.int64)                           # tokens cached per slot

    # ---- pages of a slot --------------------------------------------------------------------------
    def _sync_row(self, slot: int):
        row = self.table_host[slot]
        row[:] = 0
        row[:len(self.owned[slot])] = self.owned[slot]
        self.table[slot].copy_(torch.from_numpy(row), non_blocking=False)

    def reserve(self, slot: int, n_tokens: int):
        """Make room for ``n_tokens`` cached tokens in ``slot`` (call before a step that appends): allocates the missing pages and,
        if the page that takes the next row is still shared with a checkpoint, replaces it by a private copy."""
        assert 0 <= slot < self.S and n_tokens <= self.Lmax, (slot, n_tokens)
        P = self.pages.page_size
        own, changed = self.owned[slot], False
        cur = int(self.length[slot])
        if cur % P and cur // P < len(own) and self.pages.refs[own[cur // P]] > 1:     # appending would write into a shared page
            fresh = self.pages.alloc()
            self.pages.copy_rows(fresh, own[cur // P], cur % P)
            self.pages.release([own[cur // P]])
            own[cur // P] = fresh
            changed = True
        while len(own) * P < n_tokens:
            own.append(self.pages.alloc())
            changed = True
        if changed:
            self._sync_row(slot)

    def release(self, slot: int):
        """The sequence in ``slot`` is finished: give its page references back (pages shared with checkpoints stay alive)."""
        self.pages.release(self.owned[slot])
        self.owned[slot] = []
        self.length[slot] = 0
        self._sync_row(slot)

    # ---- admission --------------------------------------------------------------------------------
    def _load_recurrent(self, slot: int, conv: Sequence[torch.Tensor], ssm: Sequence[torch.Tensor], pos: int):
        par = pos & 1                                                # the conv window of a slot alternates between two halves
        for i, (c, s) in enumerate(zip(conv, ssm)):
            blit(self.conv[i], c.contiguous(), 3 * CD, (slot * 2 + par) * 3 * CD, 0)
            blit(self.ssm[i], s.contiguous(), HV * DV * DK, slot * HV * DV * DK, 0)

    def admit(self, slot: int, state: dict, pos: int):
        """A prefilled single-sequence state with dense K/V (``state["kv"]`` = [(K, V)] of [1, 2, L, 256], rows [0, pos) valid;
        conv [1,3,6144], ssm [1,16,128,128]) enters ``slot``: K/V rows are written into freshly allocated pages."""
        assert not self.owned[slot], "release the slot first"
        self._load_recurrent(slot, state["conv"], state["ssm"], pos)
        self.reserve(slot, pos)
        P = self.pages.page_size
        for i, page in enumerate(self.owned[slot]):
            n = min(P, pos - i * P)
            if n > 0:
                self.pages.write_rows(page, 0, state["kv"], i * P, n)
        self.length[slot] = pos

    def admit_paged(self, slot: int, live: dict, pos: int):
        """What ``PrefixCache.restore_paged`` returned enters ``slot``: the slot takes over the caller's page references (no K/V is
        moved), the recurrent state is copied into the slot pools."""
        assert not self.owned[slot], "release the slot first"
        self._load_recurrent(slot, live["conv"], live["ssm"], pos)
        self.owned[slot] = list(live["pages"])
        self.length[slot] = pos
        self._sync_row(slot)

    def checkpoint_state(self, slot: int):
        """The slot's state in the form ``PrefixCache.insert`` takes for paged sequences: its page numbers (shared, not copied, by
        the cache) and copies of the recurrent state."""
        pos = int(self.length[slot])
        par = pos & 1
        return {"pages": list(self.owned[slot]), "conv": [c[slot * 2 + par][None].clone() for c in self.conv],
                "ssm": [s[slot][None].clone() for s in self.ssm]}

    # ---- the step's operators -----------------------------------------------------------------------
    def deltanet(self, layer: int, proj, conv_w, A_log, dt_bias, slots: torch.Tensor, pos: torch.Tensor, out=None):
        """``deltanet_b`` on this pool's conv / ssm of GatedDeltaNet layer ``layer``."""
        return deltanet_b(proj, self.conv[layer], conv_w, A_log, dt_bias, self.ssm[layer], slots, pos, out=out)

    def attn(self, layer: int, q, k_new, v_new, slots: torch.Tensor, ctx_len: torch.Tensor, M: int = 1):
        """Decode attention of full-attention layer ``layer`` for the sequences in ``slots`` (int32 on the device): reads the page
        pool through the block table and appends the step's rows.  ``reserve`` must have made room for ctx_len + M tokens."""
        table = self.table.index_select(0, slots.long())
        return attn_paged(q, k_new, v_new, self.pages.K[layer], self.pages.V[layer], table, ctx_len, M=M, max_ctx=self.Lmax)

    def advance(self, slot: int, n: int):
        """Book-keeping after a step appended ``n`` rows to ``slot``."""
        self.length[slot] += n
