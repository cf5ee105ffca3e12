"""ctypes wrapper of oracle/c/libqoracle.so (the C restatement; test infrastructure only, see qoracle.c)."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "c", "libqoracle.so")
_lib = None


def build():
    subprocess.run(["make", "-C", os.path.join(HERE, "c")], check=True, capture_output=True)
    return LIB


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB):
            build()
        _lib = C.CDLL(LIB)
        _lib.qo_qmm.restype = C.c_int
        _lib.qo_moe_ffn.restype = C.c_int
    return _lib


def host_threads() -> int:
    """Hardware threads this process may run on."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def set_threads(n: int = 0) -> int:
    """Sets the OpenMP thread count of the C oracle (n <= 0: every hardware thread of the host) and returns it. Needed
    under launchers that export OMP_NUM_THREADS=1."""
    lib().qo_set_threads.restype = C.c_int
    return int(lib().qo_set_threads(C.c_int(n if n > 0 else host_threads())))


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def qmm(x, w, scales, biases, mode: str, bits: int, group: int):
    """Y = X · dequant(W)^T. x float32 [M, K]; w uint32 [N, K*bits/32]; returns (y float32 [M, N], threads)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.uint32)
    scales = np.ascontiguousarray(scales)
    biases = None if biases is None else np.ascontiguousarray(biases, dtype=np.uint16)
    M, K = x.shape
    N = w.shape[0]
    y = np.empty((M, N), dtype=np.float32)
    thr = lib().qo_qmm(_p(x), _p(w), _p(scales), _p(biases), C.c_int(1 if mode == "mxfp4" else 0), C.c_int(bits),
                       C.c_int(group), _p(y), C.c_int(M), C.c_int(N), C.c_int(K))
    return y, thr


def route(logits, E, topk, logit_bias=None, scale=1.0, per_expert_scale=None):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    T, ld = logits.shape
    inds = np.empty((T, topk), dtype=np.uint32)
    wts = np.empty((T, topk), dtype=np.float32)
    lb = None if logit_bias is None else np.ascontiguousarray(logit_bias, dtype=np.float32)
    pes = None if per_expert_scale is None else np.ascontiguousarray(per_expert_scale, dtype=np.float32)
    lib().qo_route(_p(logits), C.c_int(ld), C.c_int(T), C.c_int(E), C.c_int(topk), _p(lb), C.c_float(scale), _p(pes),
                   _p(inds), _p(wts))
    return inds, wts


def moe_ffn(x, inds, wts, gate, up, down, mode: str, act: str = "silu", limit: float = 7.0, biases=None):
    """gate/up/down = (w uint32 [E, n, k/8], scales, biases-or-None) stacked. Returns (y float32 [T, D], threads)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    T, D = x.shape
    E, I = gate[0].shape[0], gate[0].shape[1]
    topk = inds.shape[1]
    inds = np.ascontiguousarray(inds, dtype=np.uint32)
    wts = np.ascontiguousarray(wts, dtype=np.float32)
    arrs = []
    for t in (gate, up, down):
        arrs += [np.ascontiguousarray(t[0], dtype=np.uint32), np.ascontiguousarray(t[1]),
                 None if t[2] is None else np.ascontiguousarray(t[2], dtype=np.uint16)]
    bg = bu = bd = None
    if biases is not None:
        bg, bu, bd = (np.ascontiguousarray(b, dtype=np.float32) for b in biases)
    y = np.empty((T, D), dtype=np.float32)
    thr = lib().qo_moe_ffn(_p(x), C.c_int(T), C.c_int(D), C.c_int(I), C.c_int(E), C.c_int(topk), _p(inds), _p(wts),
                           *[_p(a) for a in arrs], C.c_int(1 if mode == "mxfp4" else 0),
                           C.c_int(32 if mode == "mxfp4" else 64), C.c_int(2 if act == "swiglu_oai" else 0),
                           C.c_float(limit), _p(bg), _p(bu), _p(bd), _p(y))
    return y, thr
