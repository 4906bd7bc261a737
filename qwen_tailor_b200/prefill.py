"""Prefill glue of a GatedDeltaNet layer on CUDA: drop-in for ``conv_prep`` / ``gated_norm`` of the reference's ``qwen35/prefill.py``."""
from __future__ import annotations

import torch

from . import _lib
from ._lib import check, ptr, stream_ptr
from .gated_delta import _f32
from .kernels import _rows


def conv_prep(proj, conv_state, conv_w):
    """proj [S,8224] bf16, conv_state [3,6144] (or [1,3,6144]) bf16, conv_w [6144,4,1] -> q, k, v [S,16,128] bf16 (conv + silu,
    q/k l2-normalised, q scaled by 128^-1/2) and the new conv window [3,6144] (prefill.py:160-238, 262-263)."""
    _lib.require_cuda(proj, conv_state, conv_w)
    proj, stride = _rows(proj)
    S = proj.shape[0]
    cs = conv_state.reshape(3, 6144).contiguous()
    cw = conv_w.to(torch.bfloat16).reshape(-1).contiguous()
    q, k, v = (torch.empty((S, 16, 128), dtype=torch.bfloat16, device=proj.device) for _ in range(3))
    new = torch.empty((3, 6144), dtype=torch.bfloat16, device=proj.device)
    check(_lib.load().gdn_conv_prep(ptr(proj), stride, ptr(cs), ptr(cw), ptr(q), ptr(k), ptr(v), ptr(new), S, stream_ptr(proj.device)), "conv_prep")
    return q, k, v, new


def gated_norm(y, proj, gw):
    """silu(z) * rmsnorm(y) * gw on the GDN output; y [S,16,128] or [S,2048], z = proj[:, 6144:8192] (prefill.py:241-244)."""
    _lib.require_cuda(y, proj, gw)
    proj, stride = _rows(proj)
    S = proj.shape[0]
    y2 = y.reshape(S, 2048).contiguous()
    out = torch.empty_like(y2)
    check(_lib.load().gdn_gated_norm(ptr(y2), ptr(proj), stride, ptr(_f32(gw)), ptr(out), S, stream_ptr(proj.device)), "gated_norm")
    return out
