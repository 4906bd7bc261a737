"""Chunked GatedDeltaNet prefill on CUDA: drop-in for ``gdn_chunked`` of the reference's ``qwen35/gdn_nax.py``.

The module keeps the reference's file name so that ``from <pkg>.gdn_nax import gdn_chunked`` keeps working; nothing here is
specific to Apple's NAX units.  The kernel behind it works on 64-token chunks on the tcgen05 tensor cores, keeps the fp32
state in tensor memory for the whole sequence and never materialises the reference's phase-A intermediates (Tb, Am, gv) in
device memory, so the reference's ``prep_a`` / ``phase_b`` split has no counterpart: ``gdn_chunked`` is the entry point.
``gdn_chunked_varlen`` is the additive extension for packed ragged batches and prefix-cache resume.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import check, ptr, stream_ptr
from .gated_delta import gates

FLAGS = ("RNE", "SPLIT_P1", "SPLIT_P2", "SPLIT_D", "SPLIT_Y", "SPLIT_DP", "PF")     # accepted and ignored: see gdn_chunked
DEFAULT_FLAGS = frozenset()


def gdn_chunked_varlen(q, k, v, lg, beta, cu_seqlens, init_state=None, init_idx=None, head_lo=0, head_hi=None, y=None, final_state=None):
    """Packed varlen chunked prefill.

    q, k, v: [total_T, H, 128] bf16 (q, k normalised, q scaled by 128^-1/2); lg, beta: [total_T, H] fp32 (log-decay and beta);
    cu_seqlens: int32 [n_seq + 1] on the device; init_state: fp32 [*, H, 128, 128] or None (zero states); init_idx: int32 [n_seq]
    (row of init_state each sequence resumes from, negative = zero state) or None (row s for sequence s).
    Only heads [head_lo, head_hi) are computed (head-group sharding); the rest of y / final_state is left untouched.
    Returns (y [total_T, H, 128] bf16, final_state [n_seq, H, 128, 128] fp32)."""
    _lib.require_cuda(q, k, v, lg, beta, cu_seqlens, init_state, init_idx)
    total_T, H, D = q.shape
    if D != 128 or k.shape != q.shape or v.shape != q.shape:
        raise ValueError(f"gdn_chunked: q, k, v must be [T, H, 128] with equal shapes (q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)})")
    for t in (q, k, v):
        assert t.dtype == torch.bfloat16 and t.is_contiguous()
    assert lg.dtype == torch.float32 and beta.dtype == torch.float32 and lg.is_contiguous() and beta.is_contiguous()
    assert tuple(lg.shape) == (total_T, H) and tuple(beta.shape) == (total_T, H)
    assert cu_seqlens.dtype == torch.int32 and cu_seqlens.dim() == 1
    n_seq = cu_seqlens.numel() - 1
    head_hi = H if head_hi is None else head_hi
    if init_state is not None:
        assert init_state.dtype == torch.float32 and init_state.is_contiguous() and tuple(init_state.shape[1:]) == (H, 128, 128)
    if init_idx is not None:
        assert init_idx.dtype == torch.int32 and init_idx.numel() == n_seq
    if y is None:
        y = torch.empty_like(q)
    if final_state is None:
        final_state = torch.empty((n_seq, H, 128, 128), dtype=torch.float32, device=q.device)
    check(_lib.load().gdn_prefill_chunked(ptr(q), ptr(k), ptr(v), ptr(lg), ptr(beta), ptr(cu_seqlens), ptr(init_state), ptr(init_idx), ptr(y),
                                          ptr(final_state), n_seq, total_T, H, head_lo, head_hi, stream_ptr(q.device)), "gdn_chunked")
    return y, final_state


def gdn_chunked(q, k, v, proj, A_log, dt_bias, state, relaxed=True, flags=DEFAULT_FLAGS, tg=None):
    """q,k,v [S,16,128] bf16 (q/k already normalized + scaled), proj [S,8224] bf16 (b at 8192:8208, a at 8208:8224),
    state [1,16,128,128] fp32.  Returns y [S,16,128] bf16, new_state [1,16,128,128] fp32  (gdn_nax.py:413-426).

    ``relaxed``, ``flags`` and ``tg`` tune the reference's Metal kernel (tensor-op precision switches and threadgroup size);
    they are accepted for call compatibility.  This kernel always feeds fp32-derived operands as bf16 hi + lo pairs, which
    corresponds to all SPLIT_* flags being on."""
    S = q.shape[0]
    assert proj.dtype == torch.bfloat16 and proj.dim() == 2 and proj.shape[0] == S and proj.shape[1] >= 8224 and proj.stride(1) == 1
    _, lg, beta = gates(proj[:, 8208:8224], proj[:, 8192:8208], A_log, dt_bias)
    cu = torch.tensor([0, S], dtype=torch.int32, device=q.device)
    y, st = gdn_chunked_varlen(q.contiguous(), k.contiguous(), v.contiguous(), lg, beta, cu, init_state=state.contiguous())
    return y, st
