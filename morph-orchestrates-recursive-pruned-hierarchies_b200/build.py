"""Builds libmortar_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python morph-orchestrates-recursive-pruned-hierarchies_b200/build.py [--force] [--verbose]
"""
from __future__ import annotations

import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libmortar_b200.so")
SOURCES = ["host_pack.cpp", "prefill_sched.cpp", "stream_kernels.cu", "prefill_tc.cu", "stack_decode.cu",
           "router.cu", "backward.cu", "backward_tc.cu", "gemv_tc.cu"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


OBJ = os.path.join(PKG, "_build")            # per-source objects (ignored by git; only the .so is used)


def _deps_mtime(src: str) -> float:
    """A source is rebuilt when it, any header beside it or the public header is newer than its object."""
    paths = [os.path.join(CSRC, src), os.path.join(ROOT, "include", "mortar_b200.h")]
    paths += [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    return max(os.path.getmtime(p) for p in paths)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every source under csrc/ (in parallel, one object each) and link one shared library;
    returns its path."""
    from concurrent.futures import ThreadPoolExecutor
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    os.makedirs(OBJ, exist_ok=True)
    base = [nvcc, "-O3", "-std=c++17", "-lineinfo", *ARCH, "-Xcompiler", "-fPIC",
            "-I", os.path.join(ROOT, "include"), "-I", CSRC]
    if verbose:
        base += ["-Xptxas", "-v"]

    def compile_one(src: str):
        obj = os.path.join(OBJ, src + ".o")
        if not force and os.path.exists(obj) and os.path.getmtime(obj) >= _deps_mtime(src):
            return obj, False
        cmd = base + ["-c", os.path.join(CSRC, src), "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed ({res.returncode}): {' '.join(cmd)}")
        return obj, True

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        results = list(pool.map(compile_one, SOURCES))
    objs = [o for o, _ in results]
    if any(changed for _, changed in results) or not os.path.exists(LIB) or \
            os.path.getmtime(LIB) < max(os.path.getmtime(o) for o in objs):
        cmd = [nvcc, *ARCH, "-shared", "-Xcompiler", "-fPIC", *objs, "-o", LIB]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError(f"link failed ({res.returncode}): {' '.join(cmd)}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
