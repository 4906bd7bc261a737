"""Batched decode building blocks on CUDA: drop-in for the operators and pools of the reference's ``qwen35/batch.py``.

State lives in slot pools that the kernels update in place (reference layout, batch.py:1-17):
  ssm  : n_linear x [S+1, 16, 128, 128] fp32      slot s = one sequence
  conv : n_linear x [(S+1)*2, 3, 6144]  bf16      double buffered: a step reads buffer pos&1 and writes the other one
  K, V : n_full   x [S+1, 2, Lmax, 256] bf16      the attention kernel appends each sequence's new row at its position
  slot S is a trash slot that the padding rows of a bucketed batch point at.
In-place writes are ordered against later readers by CUDA stream order.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import check, ptr, stream_ptr
from .config import Cfg
from .gated_delta import _f32
from .kernels import _rows

HV, DK, DV, CD, PW = 16, 128, 128, 6144, 8224


def deltanet_b(proj, conv_pool, conv_w, A_log, dt_bias, ssm_pool, slots, pos, out=None):
    """proj [B, 8224] bf16; slots / pos int32 [B] (pos = tokens already in the slot's state).  Returns y [B, 2048] bf16 and updates
    ssm_pool[slot] and the conv buffer (pos&1)^1 of the slot IN PLACE (batch.py:128-135).  ``out`` (optional, additive): a
    contiguous bf16 [B, 2048] tensor that receives y instead of a fresh one."""
    _lib.require_cuda(proj, conv_pool, conv_w, ssm_pool, slots, pos)
    proj, stride = _rows(proj)
    B = proj.shape[0]
    assert ssm_pool.dtype == torch.float32 and ssm_pool.is_contiguous() and conv_pool.dtype == torch.bfloat16 and conv_pool.is_contiguous()
    assert slots.dtype == torch.int32 and pos.dtype == torch.int32 and slots.numel() == B and pos.numel() == B
    if out is None:
        y = torch.empty((B, HV * DV), dtype=torch.bfloat16, device=proj.device)
    else:
        assert out.dtype == torch.bfloat16 and out.is_contiguous() and tuple(out.shape) == (B, HV * DV) and out.device == proj.device
        y = out
    cw = conv_w.to(torch.bfloat16).reshape(-1).contiguous()
    check(_lib.load().gdn_deltanet_b(ptr(proj), stride, ptr(conv_pool), ptr(cw), ptr(_f32(A_log)), ptr(_f32(dt_bias)), ptr(ssm_pool),
                                     ptr(slots), ptr(pos), ssm_pool.shape[0], ptr(y), B, stream_ptr(proj.device)), "deltanet_b")
    return y


def attn_paged(q, k_new, v_new, k_pages, v_pages, block_table, ctx_len, M=1, max_ctx=None):
    """GQA decode attention over a paged KV cache (no counterpart in the reference, whose K/V pools are contiguous per slot).

    q [R,8,256], k_new / v_new [R,2,256] bf16 (normed + roped), R = B*M; pages [n_pages, 2, page_size, 256] bf16;
    block_table int32 [B, max_pages]; ctx_len int32 [B] = tokens already cached.  Row b*M+j attends the cached keys of sequence b
    and the new rows 0..j; the new rows are appended at ctx_len[b]+j (in place).  Returns o [R,8,256] bf16."""
    _lib.require_cuda(q, k_new, v_new, k_pages, v_pages, block_table, ctx_len)
    R, H, D = q.shape
    n_pages, KV, page_size, _ = k_pages.shape
    if (H, KV, D) != (8, 2, 256) or not 1 <= M <= 4 or R % M:
        raise ValueError(f"attn: only 8 query heads, 2 KV heads, head_dim 256 and 1 <= M <= 4 are supported (H={H}, KV={KV}, D={D}, M={M})")
    B = R // M
    for t in (q, k_new, v_new, k_pages, v_pages):
        assert t.dtype == torch.bfloat16 and t.is_contiguous()
    assert block_table.dtype == torch.int32 and ctx_len.dtype == torch.int32 and block_table.is_contiguous()
    max_pages = block_table.shape[1]
    if max_ctx is None:
        max_ctx = max_pages * page_size
    lib = _lib.load()
    ws = torch.empty((max(lib.gqa_decode_workspace_bytes(B, max_ctx), 16) + 3) // 4, dtype=torch.float32, device=q.device)
    o = torch.empty((R, H, D), dtype=torch.bfloat16, device=q.device)
    check(lib.gqa_decode_paged(ptr(q), ptr(k_new), ptr(v_new), ptr(k_pages), ptr(v_pages), ptr(block_table), ptr(ctx_len), ptr(o), ptr(ws),
                               ws.numel() * 4, B, M, page_size, max_pages, n_pages, max_ctx, stream_ptr(q.device)), "attn")
    return o


def attn_paged_static(q, k_new, v_new, k_pages, v_pages, block_table, ctx_len, M=1, max_ctx=None):
    """``attn_paged`` without any allocation on the way to the kernel except the output tensor: the split-KV partials go to a
    12 MiB scratch array built into the library instead of a torch workspace.  Meant for hosts that may not allocate device
    memory while serving (their C callers pass a preallocated output and use the C entry point ``gqa_decode_paged_static``
    directly).  Raises ValueError for more than 256 sequences per call (what the array is sized for).  Calls that overlap on one
    GPU share the array and must not run concurrently; the first call on a device should happen outside stream capture."""
    _lib.require_cuda(q, k_new, v_new, k_pages, v_pages, block_table, ctx_len)
    R, H, D = q.shape
    n_pages, KV, page_size, _ = k_pages.shape
    if (H, KV, D) != (8, 2, 256) or not 1 <= M <= 4 or R % M:
        raise ValueError(f"attn: only 8 query heads, 2 KV heads, head_dim 256 and 1 <= M <= 4 are supported (H={H}, KV={KV}, D={D}, M={M})")
    B = R // M
    for t in (q, k_new, v_new, k_pages, v_pages):
        assert t.dtype == torch.bfloat16 and t.is_contiguous()
    assert block_table.dtype == torch.int32 and ctx_len.dtype == torch.int32 and block_table.is_contiguous()
    max_pages = block_table.shape[1]
    if max_ctx is None:
        max_ctx = max_pages * page_size
    o = torch.empty((R, H, D), dtype=torch.bfloat16, device=q.device)
    check(_lib.load().gqa_decode_paged_static(ptr(q), ptr(k_new), ptr(v_new), ptr(k_pages), ptr(v_pages), ptr(block_table), ptr(ctx_len), ptr(o),
                                              B, M, page_size, max_pages, n_pages, max_ctx, stream_ptr(q.device)), "attn (static scratch)")
    return o


def attn_b(q, k, v, Kp, Vp, slots, pos, M=1):
    """q [R,H,D], k / v [R,KV,D] (normed + roped), pools [S+1,KV,Lmax,D]; R = B*M rows (row b*M+j = position pos[b]+j of slot
    slots[b]; slots / pos int32 [B]).  Returns o [R,H,D] bf16 and appends k / v at pos[b]+j (in place)  (batch.py:230-237).
    The slot pool is a paged cache with one page of Lmax rows per sequence."""
    return attn_paged(q, k, v, Kp, Vp, slots.reshape(-1, 1), pos, M=M, max_ctx=Kp.shape[2])


def blit(dst, src, n, d0, s0, ny=1, dstride=0, sstride=0):
    """dst.flat[d0 + y*dstride + i] = src.flat[s0 + y*sstride + i]  for i < n, y < ny   (in place; batch.py:367-372).
    Returns dst (the reference returns a token to evaluate; stream order plays that role here)."""
    _lib.require_cuda(dst, src)
    assert dst.dtype == src.dtype and dst.dtype in (torch.bfloat16, torch.float32), (dst.dtype, src.dtype)
    assert dst.is_contiguous() and src.is_contiguous()
    assert d0 + (ny - 1) * dstride + n <= dst.numel() and s0 + (ny - 1) * sstride + n <= src.numel(), "blit out of range"
    check(_lib.load().gdn_state_copy(ptr(dst), ptr(src), dst.element_size(), n, d0, s0, ny, dstride, sstride, stream_ptr(dst.device)), "blit")
    return dst


def hrec(hist, Hn, slots, pos):
    """hist[slots[b], pos[b], :] = Hn[b]  (in place; hist [S+1, Lh, H] bf16): the hidden-state history of speculative mode
    (batch.py:375-399).  slots, pos: int32 [B] on the device; an out-of-range entry skips its row and sets the device status.
    Returns hist (the reference returns a token to evaluate; here stream order does that job)."""
    _lib.require_cuda(hist, Hn, slots, pos)
    assert hist.dtype == torch.bfloat16 and Hn.dtype == torch.bfloat16 and hist.is_contiguous() and hist.dim() == 3
    assert slots.dtype == torch.int32 and pos.dtype == torch.int32
    Hn = Hn.contiguous()
    B, H = Hn.shape
    assert hist.shape[2] == H and slots.numel() == B and pos.numel() == B
    check(_lib.load().gdn_hrec(ptr(hist), ptr(Hn), ptr(slots), ptr(pos), B, hist.shape[0], hist.shape[1], H, stream_ptr(hist.device)), "hrec")
    return hist


class Pools:
    """Slot pools of the batched decode step (batch.py:405-462)."""

    def __init__(self, cfg: Cfg, slots: int, max_len: int, device="cuda"):
        self.cfg, self.S, self.Lmax = cfg, slots, max_len
        nl, na = cfg.n_linear, cfg.n_full
        self.conv = [torch.zeros(((slots + 1) * 2, 3, CD), dtype=torch.bfloat16, device=device) for _ in range(nl)]
        self.ssm = [torch.zeros((slots + 1, HV, DV, DK), dtype=torch.float32, device=device) for _ in range(nl)]
        self.K = [torch.zeros((slots + 1, cfg.n_kv, max_len, cfg.head_dim), dtype=torch.bfloat16, device=device) for _ in range(na)]
        self.V = [torch.zeros((slots + 1, cfg.n_kv, max_len, cfg.head_dim), dtype=torch.bfloat16, device=device) for _ in range(na)]

    def nbytes(self):
        return sum(a.numel() * a.element_size() for g in (self.conv, self.ssm, self.K, self.V) for a in g)

    @staticmethod
    def slot_bytes(cfg: Cfg, max_len: int, double_conv=True):
        """Bytes one sequence occupies in the pools (the pools hold slots + 1 of these).  double_conv=False: a stand-alone state."""
        nl, na = cfg.n_linear, cfg.n_full
        return (nl * (HV * DV * DK * 4 + (2 if double_conv else 1) * 3 * CD * 2) + na * 2 * cfg.n_kv * max_len * cfg.head_dim * 2)

    def as_tree(self):
        return {"conv": self.conv, "ssm": self.ssm, "K": self.K, "V": self.V}

    def load(self, slot: int, state: dict, pos: int):
        """Copy a prefilled single-sequence state (kv [1,2,max_len,256] pairs, conv [1,3,6144], ssm [1,16,128,128], valid after
        ``pos`` tokens) into ``slot``, in place."""
        assert 0 <= slot < self.S and 0 < pos <= self.Lmax, (slot, pos)
        par = pos & 1
        for i, (c, s) in enumerate(zip(state["conv"], state["ssm"])):
            blit(self.conv[i], c.contiguous(), CD * 3, (slot * 2 + par) * 3 * CD, 0)
            blit(self.ssm[i], s.contiguous(), HV * DV * DK, slot * HV * DV * DK, 0)
        nkv, D = self.cfg.n_kv, self.cfg.head_dim
        for i, (K, V) in enumerate(state["kv"]):
            smax = K.shape[2]
            for pool, src in ((self.K[i], K), (self.V[i], V)):
                blit(pool, src.contiguous(), pos * D, slot * nkv * self.Lmax * D, 0, ny=nkv, dstride=self.Lmax * D, sstride=smax * D)

    def read(self, slot: int, pos: int, max_len: int | None = None):
        """The slot's state as a single-sequence state dict (fresh tensors)."""
        ml = max_len or self.Lmax
        par = pos & 1
        st = {"kv": [], "conv": [self.conv[i][slot * 2 + par][None].clone() for i in range(len(self.conv))],
              "ssm": [self.ssm[i][slot][None].clone() for i in range(len(self.ssm))]}
        for K, V in zip(self.K, self.V):
            def one(Pl):
                out = torch.zeros((1, Pl.shape[1], ml, Pl.shape[3]), dtype=Pl.dtype, device=Pl.device)
                n = min(pos, ml)
                out[0, :, :n] = Pl[slot, :, :n]
                return out
            st["kv"].append((one(K), one(V)))
        return st
