"""Compile the C restatement of the oracle (oracle/gdn_oracle.c) into oracle/_build/libgdn_oracle.so and bind it with ctypes.

Test infrastructure only.  The reference itself has no C/C++ sources (all of its kernels are Metal strings inside Python
files), so there is nothing to compile into oracle/_ref."""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
SRC = HERE / "gdn_oracle.c"
OUT = HERE / "_build" / "libgdn_oracle.so"


def build(force: bool = False) -> Path:
    if OUT.exists() and not force and OUT.stat().st_mtime >= SRC.stat().st_mtime:
        return OUT
    OUT.parent.mkdir(exist_ok=True)
    cmd = ["gcc", "-O3", "-march=x86-64-v3", "-fopenmp", "-shared", "-fPIC", "-o", str(OUT), str(SRC), "-lm"]
    subprocess.run(cmd, check=True)
    return OUT


_lib = None


def load():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(str(build()))
        _lib.oracle_max_threads.restype = ctypes.c_int
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def deltanet_b(proj_bits, conv_pool_bits, conv_w_bits, A_log, dt_bias, ssm_pool, slots, pos):
    """In-place decode step on numpy arrays (bf16 tensors as uint16 bit patterns).  Returns y bits [B, 2048]."""
    B = proj_bits.shape[0]
    y = np.empty((B, 2048), np.uint16)
    load().oracle_deltanet_b(_p(proj_bits), _p(conv_pool_bits), _p(conv_w_bits), _p(A_log), _p(dt_bias), _p(ssm_pool), _p(slots), _p(pos),
                             _p(y), ctypes.c_int(B))
    return y


def gated_delta_rule(q_bits, k_bits, v_bits, g, beta, S):
    """Sequential rule, fp32, S [B,H,128,128] updated in place.  Returns y bits [B,T,H,128]."""
    B, T, H, _ = q_bits.shape
    y = np.empty((B, T, H, 128), np.uint16)
    load().oracle_gated_delta_rule(_p(q_bits), _p(k_bits), _p(v_bits), _p(g), _p(beta), _p(S), _p(y), ctypes.c_int(B), ctypes.c_int(T),
                                   ctypes.c_int(H))
    return y


def attn_row(q_bits, K_bits, V_bits):
    """One query row (8 heads) over contiguous K/V [2, n, 256].  Returns o bits [8, 256]."""
    o = np.empty((8, 256), np.uint16)
    load().oracle_attn_row(_p(q_bits), _p(K_bits), _p(V_bits), _p(o), ctypes.c_int(K_bits.shape[1]))
    return o


def max_threads() -> int:
    return int(load().oracle_max_threads())


if __name__ == "__main__":
    print(build(force=True))
