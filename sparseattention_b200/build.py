"""Builds ``libsparseattn_b200.so`` (the C-ABI library of ``include/sa_b200.h``) in-tree
with nvcc for sm_100a.  Run as ``python -m sparseattention_b200.build``.

The library links the CUDA runtime statically and resolves the one driver entry point
it needs (the tensor-map encoder) at run time, so it loads on a machine without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
INCLUDE = os.path.join(os.path.dirname(PKG_DIR), "include")
LIB_PATH = os.path.join(PKG_DIR, "libsparseattn_b200.so")
SOURCES = ["classify_sm100.cu", "attn_simt.cu", "attn_bwd_simt.cu", "attn_bwd_mma.cu", "attn_fwd_sm100.cu", "selftest_sm100.cu", "capi.cu"]
HEADERS = ["sa_common.cuh", "ptx_sm100.cuh"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: cannot build libsparseattn_b200.so")
    return cand


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS] + [os.path.join(INCLUDE, "sa_b200.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not is_stale():
        return LIB_PATH
    from concurrent.futures import ThreadPoolExecutor

    ccbin = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    common = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC", "-ccbin", ccbin, "-I", INCLUDE, "-I", CSRC]
    if verbose:
        common += ["-Xptxas", "-v"]
    obj_dir = os.path.join(PKG_DIR, "build")
    os.makedirs(obj_dir, exist_ok=True)

    def compile_one(src):
        obj = os.path.join(obj_dir, src.replace(".cu", ".o"))
        res = subprocess.run(common + ["-c", os.path.join(CSRC, src), "-o", obj], capture_output=True, text=True)
        return src, obj, res

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        results = list(pool.map(compile_one, SOURCES))
    for src, _, res in results:
        if verbose:
            sys.stderr.write(res.stdout + res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n" + res.stdout + res.stderr)
    link = [_nvcc(), "-shared", "-cudart", "static", "-ccbin", ccbin, "-o", LIB_PATH] + [o for _, o, _ in results]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("link failed:\n" + res.stdout + res.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force=True, verbose="-v" in sys.argv))
