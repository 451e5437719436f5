"""Ahead-of-time build of the sm_100a kernel library.

Every ``.cu`` under this folder is compiled with
``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo`` (cross-compiles without a GPU) and
linked into ``titan_b200/_C/libtitan_b200.so``, which `titan_b200.ops._lib` loads with ctypes.
The kernels expose a plain C API (raw pointers + a CUDA stream), so the library depends on the
CUDA runtime only and builds in seconds; objects are cached by source mtime.

Counterpart of the reference's JIT op builder (torchtitan_npu/ops/aclnn/builder.py:18-56), done
ahead of time so the built library travels with the source tree.

Usage: ``python -m titan_b200.csrc.build [--force] [--verbose]``
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
OUT_DIR = os.path.join(PKG, "_C")
OBJ_DIR = os.path.join(OUT_DIR, "obj")
LIB_PATH = os.path.join(OUT_DIR, "libtitan_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put CUDA's bin directory on PATH")


def sources() -> list[str]:
    out = []
    for root, _, files in os.walk(HERE):
        for f in sorted(files):
            if f.endswith(".cu"):
                out.append(os.path.join(root, f))
    return sorted(out)


def _headers_mtime() -> float:
    m = 0.0
    for root, _, files in os.walk(HERE):
        for f in files:
            if f.endswith((".cuh", ".h")):
                m = max(m, os.path.getmtime(os.path.join(root, f)))
    return m


def _obj_for(src: str) -> str:
    rel = os.path.relpath(src, HERE).replace(os.sep, "__")
    return os.path.join(OBJ_DIR, rel[:-3] + ".o")


def _compile(src: str, verbose: bool) -> str:
    obj = _obj_for(src)
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", HERE, "-c", src, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        print(res.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile what is stale, link, and return the library path."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    srcs = sources()
    hdr = _headers_mtime()
    stale = []
    for s in srcs:
        o = _obj_for(s)
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr):
            stale.append(s)
    if stale:
        with ThreadPoolExecutor(max_workers=min(8, len(stale))) as ex:
            list(ex.map(lambda s: _compile(s, verbose), stale))
    objs = [_obj_for(s) for s in srcs]
    need_link = force or stale or not os.path.exists(LIB_PATH) or any(
        os.path.getmtime(o) > os.path.getmtime(LIB_PATH) for o in objs)
    if need_link:
        cmd = [_nvcc(), "-shared", "-o", LIB_PATH, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
