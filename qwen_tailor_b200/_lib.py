"""ctypes binding of libgdn_b200.so (the C ABI declared in include/gdn_b200.h).

There is no CPU or PyTorch fallback: if the library is missing it is built with nvcc on first use, and if that is not
possible every operator raises.  Tensors cross the boundary as raw device pointers.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_longlong, c_size_t, c_void_p, POINTER

from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent
_LIB_PATH = _PKG / "libgdn_b200.so"
_lib = None

ERRORS = {-1: "shape", -2: "dtype", -3: "alignment", -4: "index", -5: "launch", -6: "timeout", -7: "unsupported", -8: "null pointer"}

P, LL, I, F, SZ = c_void_p, c_longlong, c_int, c_float, c_size_t

# name -> (restype, argtypes); must list every symbol of include/gdn_b200.h
SIGNATURES = {
    "gdn_version": (I, []),
    "gdn_last_error_string": (c_char_p, []),
    "gdn_device_status": (I, [POINTER(c_int)]),
    "gdn_gates": (I, [P, P, LL, LL, P, P, P, P, P, LL, I, P]),
    "gdn_normalize_qk": (I, [P, P, P, P, LL, F, F, P]),
    "gdn_recurrent": (I, [P, P, P, P, P, P, P, P, I, I, I, I, I, I, P]),
    "gdn_prefill_chunked": (I, [P, P, P, P, P, P, P, P, P, P, P, SZ, I, LL, I, I, I, P]),
    "gdn_prefill_workspace_bytes": (SZ, [I, LL, I]),
    "gdn_phase_a": (I, [P, P, P, P, P, SZ, I, LL, I, I, I, P]),
    "gdn_prep_a": (I, [P, LL, P, P, P, P, P, P, P, P, P, SZ, I, LL, I, I, P]),
    "gdn_phase_b": (I, [P, P, P, P, SZ, P, P, P, P, P, I, LL, I, I, I, P]),
    "gdn_phase_b_gated": (I, [P, P, P, P, SZ, P, P, P, P, LL, P, P, P, I, LL, I, I, I, P]),
    "gdn_deltanet": (I, [P, LL, P, P, P, P, P, P, I, P, P, P, I, P]),
    "gdn_deltanet_b": (I, [P, LL, P, P, P, P, P, P, P, I, P, I, P]),
    "gdn_deltanet_bm": (I, [P, LL, P, P, P, P, P, P, P, P, I, P, I, I, P]),
    "gqa_decode_workspace_bytes": (SZ, [I, I]),
    "gqa_decode_paged": (I, [P, P, P, P, P, P, P, P, P, SZ, I, I, I, I, I, I, P]),
    "gqa_decode_paged_static": (I, [P, P, P, P, P, P, P, P, I, I, I, I, I, I, P]),
    "gqa_qkv_prep": (I, [P, LL, P, P, P, P, P, P, P, I, F, F, P]),
    "gqa_gate_out": (I, [P, P, P, LL, P]),
    "gqa_prefill_attn": (I, [P, P, P, P, I, I, LL, LL, LL, LL, P, SZ, P]),
    "gqa_prefill_attn_workspace_bytes": (SZ, [I, I]),
    "gdn_conv_prep": (I, [P, LL, P, P, P, P, P, P, I, P]),
    "gdn_gated_norm": (I, [P, P, LL, P, P, LL, P]),
    "gdn_state_copy": (I, [P, P, I, LL, LL, LL, I, LL, LL, P]),
    "gdn_hrec": (I, [P, P, P, P, I, I, I, I, P]),
}


def lib_path() -> Path:
    return _LIB_PATH


def load(build_if_missing: bool = True):
    """Load (building first if needed) the shared library and declare its prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        if not build_if_missing:
            raise RuntimeError(f"{_LIB_PATH} is missing; run `python -m qwen_tailor_b200.build`")
        from . import build as _build
        _build.build()
    lib = ctypes.CDLL(str(_LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)              # AttributeError here = the library does not export what the header declares
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(rc: int, what: str):
    """Map a negative return code to the exception the reference raises for the same mistake."""
    if rc == 0:
        return
    msg = load().gdn_last_error_string().decode("utf-8", "replace")
    text = f"{what}: {ERRORS.get(rc, rc)} error: {msg}"
    if rc in (-1, -2, -3, -7):
        raise ValueError(text)               # unsupported shapes raise ValueError in the reference (qwen35/gated_delta.py:164-166)
    raise RuntimeError(text)


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else c_void_p(t.data_ptr())


def stream_ptr(device=None):
    return c_void_p(torch.cuda.current_stream(device).cuda_stream)


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("qwen_tailor_b200 operators run on CUDA tensors only (there is no CPU path)")


def device_status() -> int:
    """Read and clear the device status word (1 = a kernel skipped a row because of an out-of-range index)."""
    out = c_int(0)
    check(load().gdn_device_status(ctypes.byref(out)), "gdn_device_status")
    return out.value
