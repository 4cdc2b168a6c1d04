"""Builds ``libnanopd_b200.so`` in-tree with nvcc for sm_100a (cross-compiles without a GPU).

Run as ``python -m nanopd_b200._build``; ``__graft_entry__.build()`` calls :func:`build`.
The reference builds its extension with torch's CUDAExtension and ``-arch=native``
(nanoPD/paged_attention/setup.py:5-27); this library has no torch or pybind11 in it, so a
plain nvcc command is enough and the result loads with ctypes.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libnanopd_b200.so"
SOURCES = ["capi.cu", "kv_store.cu", "decode_attention.cu", "prefill_attention.cu", "kv_migrate.cu",
           "qk_rope_store.cu", "top_k_sample.cu"]
HEADERS = [CSRC / "npd_common.cuh", PKG_DIR.parent / "include" / "nanopd_b200.h",
           PKG_DIR.parent / "include" / "nanopd_b200_testing.h"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-cudart", "static",
]
# --use_fast_math only where it was measured to pay and no result is pinned bit for bit against a library: the two
# attention kernels (their exponentials are explicit ex2.approx anyway).  The sampler's softmax and the norm/rotary
# kernel are compared with torch / transformers element by element and keep IEEE division, expf and sqrt.
FAST_MATH_SOURCES = {"decode_attention.cu", "prefill_attention.cu"}


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC or put it on PATH)")


def _stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    deps = [CSRC / s for s in SOURCES] + HEADERS + [Path(__file__)]
    return any(d.stat().st_mtime > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every .cu to an object (in parallel) and link the shared library."""
    if not force and not _stale():
        return LIB_PATH
    nvcc = _nvcc()
    obj_dir = PKG_DIR / "build"
    obj_dir.mkdir(exist_ok=True)
    procs = []
    for src in SOURCES:
        obj = obj_dir / (src + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *(["--use_fast_math"] if src in FAST_MATH_SOURCES else []),
               "-c", str(CSRC / src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    objs = []
    for src, obj, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out}")
        if verbose and out:
            print(out)
        objs.append(str(obj))
    link = [nvcc, "-shared", "-cudart", "static", "-o", str(LIB_PATH), *objs]
    res = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}")
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
