"""Ops-level gated delta rule on CUDA: drop-in for the reference's ``qwen35/gated_delta.py``.

Same names, argument order, shapes, dtypes and error behaviour; tensors are ``torch.Tensor`` on a CUDA device and the
work is done by libgdn_b200 (hand-written sm_100a kernels).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import check, ptr, stream_ptr


def _f32(x):
    return x if x.dtype == torch.float32 and x.is_contiguous() else x.float().contiguous()


def compute_g(A_log, a, dt_bias):
    """decay g = exp(-exp(A_log) * softplus(a + dt_bias)), fp32, shape of ``a`` (reference: gated_delta.py:16-18).
    ``a + dt_bias`` and the softplus are evaluated with bf16 rounding after every op, as MLX does on bf16 arrays."""
    _lib.require_cuda(a)
    a = a.to(torch.bfloat16).contiguous()
    H = a.shape[-1]
    g = torch.empty(a.shape, dtype=torch.float32, device=a.device)
    check(_lib.load().gdn_gates(ptr(a), None, H, 0, ptr(_f32(A_log)), ptr(_f32(dt_bias)), ptr(g), None, None, a.numel() // H, H,
                                stream_ptr(a.device)), "compute_g")
    return g


def gates(a, b, A_log, dt_bias):
    """(g, log-decay, beta) fp32 for bf16 ``a``, ``b`` of shape [..., H] that may be strided views of the in_proj output."""
    _lib.require_cuda(a, b)
    H = a.shape[-1]
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.stride(-1) == 1 and b.stride(-1) == 1
    a2, b2 = a.reshape(-1, H) if a.is_contiguous() else a, b.reshape(-1, H) if b.is_contiguous() else b
    assert a2.dim() == 2 and b2.dim() == 2, "strided gate inputs must be 2-D"
    n = a2.shape[0]
    g = torch.empty((n, H), dtype=torch.float32, device=a.device)
    lg = torch.empty_like(g)
    beta = torch.empty_like(g)
    check(_lib.load().gdn_gates(ptr(a2), ptr(b2), a2.stride(0), b2.stride(0), ptr(_f32(A_log)), ptr(_f32(dt_bias)), ptr(g), ptr(lg),
                                ptr(beta), n, H, stream_ptr(a.device)), "gates")
    shp = tuple(a.shape)
    return g.view(shp), lg.view(shp), beta.view(shp)


def normalize_qk(q, k, *, inv_scale: float, eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """L2-normalise q / k over the last dim (128) and fold the head_dim**-0.5 readout scale into q (gated_delta.py:21-30)."""
    _lib.require_cuda(q, k)
    if q.shape[-1] != 128 or k.shape[-1] != 128 or q.shape != k.shape:
        raise ValueError(f"normalize_qk: only head dim 128 with equal q / k shapes is supported (q {tuple(q.shape)}, k {tuple(k.shape)})")
    q = q.to(torch.bfloat16).contiguous()
    k = k.to(torch.bfloat16).contiguous()
    qo, ko = torch.empty_like(q), torch.empty_like(k)
    check(_lib.load().gdn_normalize_qk(ptr(q), ptr(k), ptr(qo), ptr(ko), q.numel() // 128, float(inv_scale), float(eps),
                                       stream_ptr(q.device)), "normalize_qk")
    return qo, ko


def gated_delta_update(q, k, v, a, b, A_log, dt_bias, state: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Gated delta rule recurrence over T tokens (gated_delta.py:143-174).

    q, k: [B, T, Hk, Dk] (already through ``normalize_qk``); v: [B, T, Hv, Dv]; a, b: [B, T, Hv]; state: [B, Hv, Dv, Dk] fp32
    (zeros if None).  Returns (y [B, T, Hv, Dv] in q's dtype, new state).  Raises ValueError outside the supported case
    (Dk = 128, fp32 state), like the reference."""
    _lib.require_cuda(q, k, v, a, b, state)
    B, T, Hk, Dk = k.shape
    Hv, Dv = v.shape[2:]
    if state is not None and state.dtype != torch.float32:
        raise ValueError(f"only the scalar-gate, Dk=128, fp32-state case is supported (state {state.dtype})")
    if Dk != 128 or Dv % 16 or Hv % Hk:
        raise ValueError(f"only the scalar-gate, Dk=128, fp32-state case is supported (Dk={Dk}, Dv={Dv})")
    q = q.to(torch.bfloat16).contiguous()
    k = k.to(torch.bfloat16).contiguous()
    v = v.to(torch.bfloat16).contiguous()
    g, _, beta = gates(a.to(torch.bfloat16).contiguous(), b.to(torch.bfloat16).contiguous(), A_log, dt_bias)
    y = torch.empty((B, T, Hv, Dv), dtype=torch.bfloat16, device=q.device)
    out = torch.empty((B, Hv, Dv, Dk), dtype=torch.float32, device=q.device)
    st = None if state is None else state.contiguous()
    check(_lib.load().gdn_recurrent(ptr(q), ptr(k), ptr(v), ptr(g), ptr(beta), ptr(st), ptr(y), ptr(out), B, T, Hk, Hv, Dk, Dv,
                                    stream_ptr(q.device)), "gated_delta_update")
    return y, out
