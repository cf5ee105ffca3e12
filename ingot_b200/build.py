"""Builds libingot_qmm.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m ingot_b200.build          # incremental
    python -m ingot_b200.build --force  # rebuild everything

The objects and the shared library land in ingot_b200/lib/ (git-ignored). Nothing else is needed at run time: the
Python side loads the library with ctypes.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIBDIR, "libingot_qmm.so")
SOURCES = ["api.cu", "qmv.cu", "moe.cu", "qmm.cu", "ep.cu", "colsplit.cu", "loader.cu", "sample.cu", "embed.cu", "tern.cu", "w8a8.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA library cannot be built")
    return exe


def _deps_newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(HERE, "..", "include", "ingot_qmm.h"))
    return hs


def _compile(src: str, force: bool, verbose: bool) -> str:
    obj = os.path.join(LIBDIR, os.path.splitext(src)[0] + ".o")
    path = os.path.join(CSRC, src)
    if force or _deps_newer(obj, [path] + _headers()):
        cmd = [nvcc(), *NVCC_FLAGS, "-c", path, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIBDIR, exist_ok=True)
    srcs = [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile(s, force, verbose), srcs))
    if force or _deps_newer(LIB, objs):
        cmd = [nvcc(), "-shared", "-o", LIB, *objs]
        nccl = os.environ.get("INGOT_NCCL_LIB")
        if nccl:
            cmd += [nccl]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
