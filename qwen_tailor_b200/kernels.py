"""Solo decode / speculative-verify operator: drop-in for ``deltanet`` of the reference's ``qwen35/kernels.py``."""
from __future__ import annotations

import torch

from . import _lib
from ._lib import check, ptr, stream_ptr
from .gated_delta import _f32

HV, DK, DV, CD, PW = 16, 128, 128, 6144, 8224


def _rows(proj):
    assert proj.dtype == torch.bfloat16 and proj.dim() == 2 and proj.shape[1] >= PW and proj.stride(1) == 1, \
        f"proj must be bf16 [rows, >=8224] with unit inner stride, got {tuple(proj.shape)} {proj.dtype}"
    return proj, proj.stride(0)


def deltanet(proj, conv_snap, conv_w, A_log, dt_bias, ssm_snap, sel):
    """proj [M, 8224] bf16 (qkv 6144 | z 2048 | b 16 | a 16 per token).
    conv_snap [S,3,6144] / ssm_snap [S,16,128,128]: state snapshots; the kernel starts from snapshot sel[0] (int32 [1] tensor).
    Returns y [M,2048], conv snapshots [M,3,6144] (after each token), ssm snapshots [M,16,128,128]  (kernels.py:555-567)."""
    _lib.require_cuda(proj, conv_snap, conv_w, ssm_snap, sel)
    proj, stride = _rows(proj)
    M = proj.shape[0]
    assert ssm_snap.dtype == torch.float32 and conv_snap.dtype == torch.bfloat16 and sel.dtype == torch.int32
    conv_snap, ssm_snap = conv_snap.contiguous(), ssm_snap.contiguous()
    S = ssm_snap.shape[0]
    dev = proj.device
    y = torch.empty((M, HV * DV), dtype=torch.bfloat16, device=dev)
    cs = torch.empty((M, 3, CD), dtype=torch.bfloat16, device=dev)
    st = torch.empty((M, HV, DV, DK), dtype=torch.float32, device=dev)
    cw = conv_w.to(torch.bfloat16).reshape(-1).contiguous()
    check(_lib.load().gdn_deltanet(ptr(proj), stride, ptr(conv_snap), ptr(cw), ptr(_f32(A_log)), ptr(_f32(dt_bias)), ptr(ssm_snap),
                                   ptr(sel), S, ptr(y), ptr(cs), ptr(st), M, stream_ptr(dev)), "deltanet")
    return y, cs, st
