"""Chunked GatedDeltaNet prefill on CUDA: drop-in for ``prep_a`` / ``phase_b`` / ``gdn_chunked`` of the reference's
``qwen35/gdn_nax.py``.

The module keeps the reference's file name so that ``from <pkg>.gdn_nax import prep_a, phase_b, gdn_chunked`` keeps working;
nothing here is specific to Apple's NAX units.  Same two-phase structure as the reference, on 64-token chunks and the tcgen05
tensor cores:

* phase A (one independent tile per (chunk, head), fills the GPU even for one sequence): cumulative decay, K K^T, the exact
  inverse (I + L)^-1, Tb = T diag(beta); ``prep_a`` fuses the conv + silu + q/k l2norm + gates front end into it
  (gdn_nax.py:394-401);
* phase B (serial over the chunks of a (sequence, head), fp32 state resident in tensor memory): ``phase_b`` (gdn_nax.py:404-410).

What travels between the phases differs from the reference's ``Tb, Am [NC,16,256] f32, gv [NC,16,32] f32``: here ``Tb`` is a byte
tensor of per-(chunk, head) records (Tb as bf16 hi + lo tensor-core operand images, followed by the chunk's cumulative log-decay,
gamma and dec vectors), ``gv`` is the int32 ``cu_seqlens`` the records were laid out by, and ``Am`` is empty: the A matrix is formed
inside phase B from Q K^T, which costs nothing there and halves what phase A writes.  Callers that only pass the tuple through, as
the reference's prefill does (qwen35/prefill.py:252-253), need no change.
``gdn_chunked_varlen`` is the additive extension for packed ragged batches and prefix-cache resume.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import check, ptr, stream_ptr
from .gated_delta import _f32, gates

FLAGS = ("RNE", "SPLIT_P1", "SPLIT_P2", "SPLIT_D", "SPLIT_Y", "SPLIT_DP", "PF")     # accepted and ignored: see gdn_chunked
DEFAULT_FLAGS = frozenset()
REC_BYTES = 17152


def records_bytes(n_seq: int, total_T: int, H: int = 16) -> int:
    """Size of the phase-A record buffer of a packed batch (what ``gdn_prefill_workspace_bytes`` returns)."""
    return int(_lib.load().gdn_prefill_workspace_bytes(n_seq, total_T, H))


def _records(n_seq, total_T, H, device):
    return torch.empty((max(records_bytes(n_seq, total_T, H), 16),), dtype=torch.uint8, device=device)


def _check_qkv(q, k, v):
    total_T, H, D = q.shape
    if D != 128 or k.shape != q.shape or v.shape != q.shape:
        raise ValueError(f"gdn_chunked: q, k, v must be [T, H, 128] with equal shapes (q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)})")
    for t in (q, k, v):
        assert t.dtype == torch.bfloat16 and t.is_contiguous()
    return total_T, H


def phase_a_varlen(k, lg, beta, cu_seqlens, head_lo=0, head_hi=None, records=None):
    """Phase A over a packed batch.  k [total_T, H, 128] bf16 (normalised), lg / beta [total_T, H] fp32, cu_seqlens int32 [n_seq + 1].
    Returns the record buffer (uint8) that ``phase_b_varlen`` consumes."""
    _lib.require_cuda(k, lg, beta, cu_seqlens)
    total_T, H, D = k.shape
    assert D == 128 and k.dtype == torch.bfloat16 and k.is_contiguous()
    assert lg.dtype == torch.float32 and beta.dtype == torch.float32 and lg.is_contiguous() and beta.is_contiguous()
    assert tuple(lg.shape) == (total_T, H) and tuple(beta.shape) == (total_T, H)
    assert cu_seqlens.dtype == torch.int32 and cu_seqlens.dim() == 1
    n_seq = cu_seqlens.numel() - 1
    head_hi = H if head_hi is None else head_hi
    if records is None:
        records = _records(n_seq, total_T, H, k.device)
    check(_lib.load().gdn_phase_a(ptr(k), ptr(lg), ptr(beta), ptr(cu_seqlens), ptr(records), records.numel(), n_seq, total_T, H, head_lo, head_hi,
                                  stream_ptr(k.device)), "gdn_phase_a")
    return records


def _gate_args(gate_proj, gate_w, total_T, H):
    """(z pointer, row stride in elements, weight tensor) of the fused gated norm, or zeros when it is off."""
    if gate_proj is None and gate_w is None:
        return 0, 0, None
    if gate_proj is None or gate_w is None:
        raise ValueError("gdn_chunked: gate_proj and gate_w go together")
    _lib.require_cuda(gate_proj, gate_w)
    assert gate_proj.dtype == torch.bfloat16 and gate_proj.dim() == 2 and gate_proj.shape[0] == total_T and gate_proj.stride(1) == 1
    assert H == 16 and gate_proj.shape[1] >= 8192, "the z slice is columns 6144:8192 of the in_proj rows"
    gw = _f32(gate_w).reshape(-1)
    assert gw.numel() == 128
    return gate_proj.data_ptr() + 6144 * 2, gate_proj.stride(0), gw


def phase_b_varlen(q, k, v, records, cu_seqlens, init_state=None, init_idx=None, head_lo=0, head_hi=None, y=None, final_state=None,
                   gate_proj=None, gate_w=None):
    """Phase B over a packed batch: the serial chain of every (sequence, head) on the records of phase A.
    With ``gate_proj`` (the in_proj rows [total_T, >= 8192] bf16) and ``gate_w`` ([128]) the layer's gated RMSNorm is applied in the
    y store -- the same bits as ``prefill.gated_norm(y, gate_proj, gate_w)`` on the plain result (qwen35/prefill.py:253-254).
    Returns (y [total_T, H, 128] bf16, final_state [n_seq, H, 128, 128] fp32)."""
    _lib.require_cuda(q, k, v, records, cu_seqlens, init_state, init_idx)
    total_T, H = _check_qkv(q, k, v)
    assert records.dtype == torch.uint8 and records.is_contiguous()
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
    gz, gstride, gw = _gate_args(gate_proj, gate_w, total_T, H)
    check(_lib.load().gdn_phase_b_gated(ptr(q), ptr(k), ptr(v), ptr(records), records.numel(), ptr(cu_seqlens), ptr(init_state), ptr(init_idx),
                                        gz, gstride, ptr(gw), ptr(y), ptr(final_state), n_seq, total_T, H, head_lo, head_hi, stream_ptr(q.device)),
          "gdn_phase_b")
    return y, final_state


def gdn_chunked_varlen(q, k, v, lg, beta, cu_seqlens, init_state=None, init_idx=None, head_lo=0, head_hi=None, y=None, final_state=None,
                       gate_proj=None, gate_w=None):
    """Packed varlen chunked prefill (phase A, then phase B).

    q, k, v: [total_T, H, 128] bf16 (q, k normalised, q scaled by 128^-1/2); lg, beta: [total_T, H] fp32 (log-decay and beta);
    cu_seqlens: int32 [n_seq + 1] on the device; init_state: fp32 [*, H, 128, 128] or None (zero states); init_idx: int32 [n_seq]
    (row of init_state each sequence resumes from, negative = zero state) or None (row s for sequence s).
    Only heads [head_lo, head_hi) are computed (head-group sharding); the rest of y / final_state is left untouched.
    ``gate_proj`` / ``gate_w``: fuse the gated RMSNorm into the y store (see ``phase_b_varlen``).
    Returns (y [total_T, H, 128] bf16, final_state [n_seq, H, 128, 128] fp32)."""
    _lib.require_cuda(q, k, v, lg, beta, cu_seqlens, init_state, init_idx)
    total_T, H = _check_qkv(q, k, v)
    head_hi_ = H if head_hi is None else head_hi
    if not (0 <= head_lo <= head_hi_ <= H):
        raise ValueError(f"gdn_chunked: head range [{head_lo}, {head_hi_}) outside [0, {H})")
    rec = phase_a_varlen(k, lg, beta, cu_seqlens, head_lo, head_hi)
    return phase_b_varlen(q, k, v, rec, cu_seqlens, init_state, init_idx, head_lo, head_hi, y, final_state, gate_proj, gate_w)


def prep_a(proj, conv_state, conv_w, A_log, dt_bias, relaxed=True):
    """conv + silu + qk-norm and GDN phase A in one kernel (bit-identical to conv_prep followed by phase A).
    proj [S,8224] bf16, conv_state [3,6144] (or [1,3,6144]), conv_w [6144,1,4] (any shape with 6144*4 elements, flat ch*4+tap)
    -> q, k, v [S,16,128] bf16, Tb (phase-A records, uint8), Am (empty: formed inside phase_b), gv (cu_seqlens of the records)
    (gdn_nax.py:394-401).  ``relaxed`` selects a tensor-op precision mode of the reference's Metal kernel and is accepted for call
    compatibility."""
    _lib.require_cuda(proj, conv_state, conv_w)
    assert proj.dtype == torch.bfloat16 and proj.dim() == 2 and proj.shape[1] >= 8224 and proj.stride(1) == 1
    S = proj.shape[0]
    dev = proj.device
    cs = conv_state.reshape(3, 6144).to(torch.bfloat16).contiguous()
    cw = conv_w.to(torch.bfloat16).reshape(-1).contiguous()
    q, k, v = (torch.empty((S, 16, 128), dtype=torch.bfloat16, device=dev) for _ in range(3))
    cu = torch.tensor([0, S], dtype=torch.int32, device=dev)
    rec = _records(1, S, 16, dev)
    check(_lib.load().gdn_prep_a(ptr(proj), proj.stride(0), ptr(cs), ptr(cw), ptr(_f32(A_log)), ptr(_f32(dt_bias)), ptr(cu), ptr(q), ptr(k), ptr(v),
                                 ptr(rec), rec.numel(), 1, S, 0, 16, stream_ptr(dev)), "prep_a")
    Am = torch.empty((0,), dtype=torch.float32, device=dev)
    return q, k, v, rec, Am, cu


def phase_a(q, k, proj, A_log, dt_bias, relaxed=True):
    """Phase A alone on already prepared k (the first kernel of the reference's gdn_chunked, gdn_nax.py:420-422): returns (Tb, Am, gv)
    in the form described in the module docstring.  ``q`` is accepted for symmetry with the reference kernel's inputs."""
    S = k.shape[0]
    _, lg, beta = gates(proj[:, 8208:8224], proj[:, 8192:8208], A_log, dt_bias)
    cu = torch.tensor([0, S], dtype=torch.int32, device=k.device)
    rec = phase_a_varlen(k.contiguous(), lg, beta, cu)
    return rec, torch.empty((0,), dtype=torch.float32, device=k.device), cu


def phase_b(q, k, v, Tb, Am, gv, state, relaxed=True, flags=DEFAULT_FLAGS, tg=None, gate_proj=None, gate_w=None):
    """The serial state recurrence (phase B) on the outputs of phase A -> y [S,16,128] bf16, new state [1,16,128,128] fp32
    (gdn_nax.py:404-410).  ``Tb, Am, gv`` are what ``prep_a`` / ``phase_a`` returned.  ``gate_proj`` / ``gate_w`` (additive): apply the
    layer's gated RMSNorm in the y store, i.e. return what the reference's next line, ``gated_norm(out, proj, gnorm)``, would."""
    y, st = phase_b_varlen(q.contiguous(), k.contiguous(), v.contiguous(), Tb, gv, init_state=None if state is None else state.contiguous(),
                           gate_proj=gate_proj, gate_w=gate_w)
    return y, st


def gdn_chunked(q, k, v, proj, A_log, dt_bias, state, relaxed=True, flags=DEFAULT_FLAGS, tg=None):
    """q,k,v [S,16,128] bf16 (q/k already normalized + scaled), proj [S,8224] bf16 (b at 8192:8208, a at 8208:8224),
    state [1,16,128,128] fp32.  Returns y [S,16,128] bf16, new_state [1,16,128,128] fp32  (gdn_nax.py:413-426).

    ``relaxed``, ``flags`` and ``tg`` tune the reference's Metal kernel (tensor-op precision switches and threadgroup size);
    they are accepted for call compatibility.  This kernel always feeds fp32-derived operands as bf16 hi + lo pairs, which
    corresponds to all SPLIT_* flags being on."""
    S = q.shape[0]
    assert proj.dtype == torch.bfloat16 and proj.dim() == 2 and proj.shape[0] == S and proj.shape[1] >= 8224 and proj.stride(1) == 1
    Tb, Am, gv = phase_a(q, k, proj, A_log, dt_bias, relaxed)
    return phase_b(q, k, v, Tb, Am, gv, state, relaxed, flags, tg)
