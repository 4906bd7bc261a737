"""Build recipe for libgdn_b200.so (nvcc, sm_100a only, in-tree output next to this file).

Usage:  python -m qwen_tailor_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libgdn_b200.so"
SOURCES = ["c_api.cu", "gdn_decode.cu", "gdn_recurrent.cu", "gqa_decode.cu", "gqa_decode_tc.cu", "gqa_prefill_tc.cu", "state_copy.cu", "gdn_phase_a.cu", "gdn_prefill_sm100.cu",
           "attn_glue.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


def nvcc_path() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found: libgdn_b200.so cannot be built (there is no CPU fallback)")
    return cand


def sources():
    return [CSRC / s for s in SOURCES if (CSRC / s).exists()]


def stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "gdn_b200.h", Path(__file__)]
    return any(d.stat().st_mtime > t for d in deps if d.exists())


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every CUDA source for sm_100a and link the shared library.  Returns the library path."""
    if not force and not stale():
        return LIB
    nvcc = nvcc_path()
    objdir = PKG / "build"
    objdir.mkdir(exist_ok=True)
    flags = list(NVCC_FLAGS)
    if verbose:
        flags += ["-Xptxas", "-v"]
    objs = []
    procs = []
    for src in sources():
        obj = objdir / (src.stem + ".o")
        objs.append(obj)
        cmd = [nvcc, *flags, "-c", str(src), "-o", str(obj)]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"--- nvcc failed on {src.name} ---\n{out}\n")
        elif verbose or out.strip():
            sys.stderr.write(f"--- {src.name} ---\n{out}\n")
    if failed:
        raise RuntimeError("nvcc failed; see messages above")
    tmp = LIB.with_suffix(".so.tmp")
    cmd = [nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a"]
    subprocess.run(cmd, check=True)
    os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
