"""ctypes wrapper over liboracle_c.so (the C restatement).  Test / baseline infrastructure only."""
from __future__ import annotations

import ctypes
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_lib = None


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(HERE, "liboracle_c.so")
        if not os.path.exists(path):
            from . import build
            build.build()
        L = ctypes.CDLL(path)
        i64, p, f, i = ctypes.c_int64, ctypes.c_void_p, ctypes.c_float, ctypes.c_int
        L.oracle_softmax_f32.argtypes = [p, p, i64, i64, f, i, i64]
        L.oracle_norm_bf16.argtypes = [p, p, p, p, i64, i64, f, i]
        L.oracle_norm_f32.argtypes = [p, p, p, p, i64, i64, f, i]
        L.oracle_gemm_f32.argtypes = [p, p, p, i64, i64, i64, i64, i, i]
        L.oracle_gemm_bf16.argtypes = [p, p, p, i64, i64, i64, i64, i, i]
        L.oracle_num_threads.restype = i
        L.oracle_set_num_threads.argtypes = [i]
        L.oracle_set_num_threads.restype = None
        _lib = L
    return _lib


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def softmax_f32(x: np.ndarray, scale=1.0, causal=False, seq_q=None, out=None) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    cols = x.shape[-1]
    rows = x.size // cols
    y = out if out is not None else np.empty_like(x)
    lib().oracle_softmax_f32(_ptr(x), _ptr(y), rows, cols, float(scale), int(causal), int(seq_q if seq_q else (x.shape[-2] if x.ndim > 1 else rows)))
    return y


def norm(x: np.ndarray, gamma, beta, eps: float, rms: bool, out=None) -> np.ndarray:
    x = np.ascontiguousarray(x)
    cols = x.shape[-1]
    rows = x.size // cols
    y = out if out is not None else np.empty_like(x)
    fn = lib().oracle_norm_f32 if x.dtype == np.float32 else lib().oracle_norm_bf16
    fn(_ptr(x), _ptr(gamma), _ptr(beta), _ptr(y), rows, cols, float(eps), int(rms))
    return y


def gemm(a: np.ndarray, b: np.ndarray, a_k_major: bool, b_k_major: bool) -> np.ndarray:
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    batch = a.shape[0]
    m, k = (a.shape[1], a.shape[2]) if a_k_major else (a.shape[2], a.shape[1])
    n = b.shape[1] if b_k_major else b.shape[2]
    c = np.empty((batch, m, n), dtype=a.dtype)
    fn = lib().oracle_gemm_f32 if a.dtype == np.float32 else lib().oracle_gemm_bf16
    fn(_ptr(a), _ptr(b), _ptr(c), batch, m, n, k, int(a_k_major), int(b_k_major))
    return c


def num_threads() -> int:
    return lib().oracle_num_threads()


def use_all_cores() -> int:
    """One OpenMP thread per core this process may run on, whatever OMP_NUM_THREADS says; returns the count."""
    import os
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().oracle_set_num_threads(n)
    return num_threads()
