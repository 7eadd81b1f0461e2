"""ctypes access to oracle/_ref/libcacheir_ref.so (the reference's own C++/OpenMP CPU
kernels, built by oracle/Makefile). TEST / BASELINE INFRASTRUCTURE ONLY."""
from __future__ import annotations

import ctypes
from pathlib import Path

import numpy as np

LIB_PATH = Path(__file__).resolve().parent / "_ref" / "libcacheir_ref.so"
_LIB = None


def available() -> bool:
    return LIB_PATH.exists()


def _lib():
    global _LIB
    if _LIB is None:
        lib = ctypes.CDLL(str(LIB_PATH))
        f32p = ctypes.POINTER(ctypes.c_float)
        lib.cacheir_ref_simd_backend.restype = ctypes.c_char_p
        lib.cacheir_ref_rms_norm.argtypes = [f32p, f32p, f32p, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_float]
        lib.cacheir_ref_silu_mul.argtypes = [f32p, f32p, f32p, ctypes.c_size_t]
        lib.cacheir_ref_matmul_out_in.argtypes = [f32p, f32p, f32p, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_size_t]
        _LIB = lib
    return _LIB


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def simd_backend() -> str:
    return _lib().cacheir_ref_simd_backend().decode()


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(weight, dtype=np.float32)
    out = np.empty_like(x)
    _lib().cacheir_ref_rms_norm(_p(x), _p(w), _p(out), x.size // x.shape[-1], x.shape[-1], float(eps))
    return out


def silu_mul(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    g = np.ascontiguousarray(gate, dtype=np.float32)
    u = np.ascontiguousarray(up, dtype=np.float32)
    out = np.empty_like(g)
    _lib().cacheir_ref_silu_mul(_p(g), _p(u), _p(out), g.size)
    return out


def matmul_out_in(x: np.ndarray, weight: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(weight, dtype=np.float32)
    rows = x.size // x.shape[-1]
    out = np.empty(x.shape[:-1] + (w.shape[0],), dtype=np.float32)
    _lib().cacheir_ref_matmul_out_in(_p(x), _p(w), _p(out), rows, x.shape[-1], w.shape[0])
    return out
