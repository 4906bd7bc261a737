"""Batched speculative verify on CUDA: drop-in for ``deltanet_bm`` / ``SpecPools`` of the reference's ``qwen35/batch_spec.py``
and for the snapshot / rollback protocol around them (qwen35/spec.py:37-65).

Snapshot pools (batch_spec.py:16-22):
  ssm  : n_linear x [NS+1, M, 16,128,128] fp32   snapshot j = state after the j-th token of the sequence's last verify; a round
                                                 starts from snapshot ``sel`` and overwrites all M snapshots in place
  conv : n_linear x [(NS+1)*2, M, 3, 6144] bf16  double buffered: a round reads buffer ``par`` and writes the other one
  entry NS is the trash entry of padded rows.
Rollback after a verify is an index choice: the next round passes ``sel = n_new``, nothing is copied.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import check, ptr, stream_ptr
from .batch import CD, DK, DV, HV, blit
from .config import Cfg
from .gated_delta import _f32
from .kernels import _rows


def deltanet_bm(proj, conv_pool, conv_w, A_log, dt_bias, ssm_pool, sslots, sels, pars, M):
    """proj [B*M, 8224] bf16 (row b*M+j = token j of sequence b); sslots / sels / pars int32 [B]: the sequence's entry in the snapshot
    pools, the snapshot it starts from, and the conv buffer it reads.  Returns y [B*M, 2048] bf16; writes snapshots 0..M-1 of
    ssm_pool[sslot] and conv buffer par^1 IN PLACE (batch_spec.py:142-150)."""
    _lib.require_cuda(proj, conv_pool, conv_w, ssm_pool, sslots, sels, pars)
    proj, stride = _rows(proj)
    B = sslots.shape[0]
    assert proj.shape[0] == B * M, (proj.shape, B, M)
    assert ssm_pool.dtype == torch.float32 and ssm_pool.is_contiguous() and ssm_pool.shape[1] == M
    assert conv_pool.dtype == torch.bfloat16 and conv_pool.is_contiguous() and conv_pool.shape[1] == M
    assert sslots.dtype == torch.int32 and sels.dtype == torch.int32 and pars.dtype == torch.int32
    y = torch.empty((B * M, HV * DV), dtype=torch.bfloat16, device=proj.device)
    cw = conv_w.to(torch.bfloat16).reshape(-1).contiguous()
    check(_lib.load().gdn_deltanet_bm(ptr(proj), stride, ptr(conv_pool), ptr(cw), ptr(_f32(A_log)), ptr(_f32(dt_bias)), ptr(ssm_pool),
                                      ptr(sslots), ptr(sels), ptr(pars), ssm_pool.shape[0], ptr(y), B, M, stream_ptr(proj.device)), "deltanet_bm")
    return y


def accept_length(toks, ids):
    """n_new [B] int32 = number of leading drafts that the verify confirmed: sum(cumprod(toks[:, 1:] == ids[:, :k]))
    (spec.py:60-61, batch_spec.py:380-381).  The result is the next round's ``sel``."""
    k = toks.shape[1] - 1
    eq = (toks[:, 1:] == ids[:, :k]).to(torch.int32)
    return torch.cumprod(eq, dim=1).sum(dim=1).to(torch.int32)


class SpecPools:
    """Recurrent snapshot pools of the sequences in speculative mode, the MTP layer's K/V pool and the round carry
    (batch_spec.py:242-270)."""

    def __init__(self, cfg: Cfg, nspec: int, nslots: int, M: int, max_len: int, device="cuda"):
        self.cfg, self.NS, self.M, self.Lmax = cfg, nspec, M, max_len
        nl = cfg.n_linear
        z = lambda shape, dt: torch.zeros(shape, dtype=dt, device=device)
        self.conv = [z(((nspec + 1) * 2, M, 3, CD), torch.bfloat16) for _ in range(nl)]
        self.ssm = [z((nspec + 1, M, HV, DV, DK), torch.float32) for _ in range(nl)]
        self.mK = z((nslots + 1, cfg.n_kv, max_len, cfg.head_dim), torch.bfloat16)
        self.mV = z((nslots + 1, cfg.n_kv, max_len, cfg.head_dim), torch.bfloat16)
        self.hist = z((nslots + 1, max_len, cfg.hidden), torch.bfloat16)
        self.carry = dict(H=z((nspec + 1, M, cfg.hidden), torch.bfloat16), toks=z((nspec + 1, M), torch.int32),
                          ids=z((nspec + 1, M), torch.int32), pos=z((nspec + 1,), torch.int32), sel=z((nspec + 1,), torch.int32))

    def as_tree(self):
        return {"conv": self.conv, "ssm": self.ssm, "mK": self.mK, "mV": self.mV}

    @staticmethod
    def entry_bytes(cfg: Cfg, M: int):
        return cfg.n_linear * M * (HV * DV * DK * 4 + 2 * 3 * CD * 2)

    @staticmethod
    def mtp_bytes(cfg: Cfg, max_len: int):
        """Per main slot: the MTP layer's K / V rows + the hidden-state history."""
        return 2 * cfg.n_kv * max_len * cfg.head_dim * 2 + max_len * cfg.hidden * 2

    # ---- moves between the plain pools and the snapshot pools (qwen35/serve.py:310-348) ----
    def enter(self, pools, slot: int, entry: int, pos: int):
        """plain -> spec: the slot's state becomes snapshot 0 / conv buffer 0 of ``entry``; the caller sets sel = 0, par = 0."""
        M = self.M
        par = pos & 1
        for i in range(len(self.ssm)):
            blit(self.ssm[i], pools.ssm[i], HV * DV * DK, entry * M * HV * DV * DK, slot * HV * DV * DK)
            blit(self.conv[i], pools.conv[i], 3 * CD, (entry * 2 + 0) * M * 3 * CD, (slot * 2 + par) * 3 * CD)

    def leave(self, pools, slot: int, entry: int, sel: int, par: int, pos: int):
        """spec -> plain: snapshot ``sel`` of ``entry`` (conv buffer ``par``) goes back into the slot, valid after ``pos`` tokens."""
        M = self.M
        for i in range(len(self.ssm)):
            blit(pools.ssm[i], self.ssm[i], HV * DV * DK, slot * HV * DV * DK, (entry * M + sel) * HV * DV * DK)
            blit(pools.conv[i], self.conv[i], 3 * CD, (slot * 2 + (pos & 1)) * 3 * CD, ((entry * 2 + par) * M + sel) * 3 * CD)
