"""The glue around the decode attention of a full-attention layer (the MLX library calls of the reference's
``qwen35/fast.py:70-85`` / ``qwen35/batch.py:504-513``) as two CUDA kernels."""
from __future__ import annotations

import torch

from . import _lib
from ._lib import check, ptr, stream_ptr
from .gated_delta import _f32


def qkv_prep(qkv, q_norm, k_norm, row_pos, eps=1e-6, rope_theta=1e7):
    """qkv [R, 5120] bf16 (8 x (q | gate), k, v) -> q [R,8,256], gate [R,2048], k [R,2,256], v [R,2,256]: q and k are
    rms-normed with q_norm / k_norm and rotated (first 64 dims, half-split pairs) at positions row_pos (int32 [R])."""
    _lib.require_cuda(qkv, q_norm, k_norm, row_pos)
    assert qkv.dtype == torch.bfloat16 and qkv.dim() == 2 and qkv.shape[1] >= 5120 and qkv.stride(1) == 1 and row_pos.dtype == torch.int32
    R = qkv.shape[0]
    dev = qkv.device
    q = torch.empty((R, 8, 256), dtype=torch.bfloat16, device=dev)
    gate = torch.empty((R, 8, 256), dtype=torch.bfloat16, device=dev)
    k = torch.empty((R, 2, 256), dtype=torch.bfloat16, device=dev)
    v = torch.empty((R, 2, 256), dtype=torch.bfloat16, device=dev)
    check(_lib.load().gqa_qkv_prep(ptr(qkv), qkv.stride(0), ptr(_f32(q_norm)), ptr(_f32(k_norm)), ptr(row_pos), ptr(q), ptr(gate), ptr(k), ptr(v), R,
                                   float(eps), float(rope_theta), stream_ptr(dev)), "qkv_prep")
    return q, gate.view(R, 2048), k, v


def gate_out(o, gate):
    """o * sigmoid(gate) with the bf16 rounding points of the unfused graph; o [R,8,256] or [R,2048], gate [R,2048]."""
    _lib.require_cuda(o, gate)
    o2 = o.reshape(o.shape[0], -1).contiguous()
    g2 = gate.reshape(o2.shape).contiguous()
    out = torch.empty_like(o2)
    check(_lib.load().gqa_gate_out(ptr(o2), ptr(g2), ptr(out), o2.numel(), stream_ptr(o.device)), "gate_out")
    return out


def prefill_attention(q, K, V, pos=0, split=True):
    """Causal attention of a prefill chunk on the tensor cores: the ``mx.fast.scaled_dot_product_attention(q, K[:, :, :kv_len],
    V[:, :, :kv_len], scale=256**-0.5, mask="causal")`` of the reference's full-attention layer (qwen35/model.py:165).

    q [S, 8, 256] bf16: the S query tokens at positions pos .. pos + S - 1 (rms-normed and rotated, as ``qkv_prep`` returns them).
    K, V: the cache including this chunk's rows, either the reference's head-major [2, T, 256] / [1, 2, T, 256] (T >= pos + S) or
    token-major [T, 2, 256]; any strides that are multiples of 8 elements with a contiguous last dimension.
    ``split`` (additive): for prefills short enough to leave at most one block per SM (about 768 to 2368 tokens from position 0) the
    query blocks with the most keys run as two blocks along the keys and are merged in the kernel (a scratch tensor is allocated);
    the launch otherwise lasts as long as its last query block.  Measured: S = 2048 53 against 61 us, S = 1024 29 against 34 us.
    Returns o [S, 8, 256] bf16."""
    _lib.require_cuda(q, K, V)
    assert q.dtype == torch.bfloat16 and q.dim() == 3 and tuple(q.shape[1:]) == (8, 256) and q.is_contiguous()
    S = q.shape[0]
    if K.dim() == 4:
        K, V = K[0], V[0]
    assert K.dtype == torch.bfloat16 and V.dtype == torch.bfloat16 and K.dim() == 3 and K.shape == V.shape and K.shape[2] == 256
    assert K.stride(2) == 1 and V.stride(2) == 1
    if K.shape[0] == 2 and K.shape[1] != 2:                         # [2, T, 256]
        T, ks, vs = K.shape[1], (K.stride(1), K.stride(0)), (V.stride(1), V.stride(0))
    elif K.shape[1] == 2:                                           # [T, 2, 256]
        T, ks, vs = K.shape[0], (K.stride(0), K.stride(1)), (V.stride(0), V.stride(1))
    else:
        raise ValueError(f"prefill_attention: K must be [2, T, 256] or [T, 2, 256], got {tuple(K.shape)}")
    if T < pos + S:
        raise ValueError(f"prefill_attention: the cache holds {T} keys, pos + S = {pos + S}")
    out = torch.empty_like(q)
    lib = _lib.load()
    ws_bytes = int(lib.gqa_prefill_attn_workspace_bytes(S, int(pos))) if split and S > 0 else 0
    ws = torch.empty((ws_bytes,), dtype=torch.uint8, device=q.device) if ws_bytes else None
    check(lib.gqa_prefill_attn(ptr(q), ptr(K), ptr(V), ptr(out), S, int(pos), ks[0], ks[1], vs[0], vs[1], ptr(ws), ws_bytes, stream_ptr(q.device)),
          "prefill_attention")
    return out
