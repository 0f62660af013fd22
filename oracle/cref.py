"""ctypes access to the plain-C oracle ``oracle/q4_ref.c`` (test infrastructure;
see ``oracle/__init__.py`` for who may import this)."""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "libq4ref.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "q4_ref.c")
    if force or not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libq4ref.so"], stdout=subprocess.DEVNULL)
    return _LIB


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.q4_dequant.restype = ctypes.c_int
        _lib.q4_dequant.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_void_p]
        _lib.q4_gemv.restype = ctypes.c_int
        _lib.q4_gemv.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]
        _lib.q4_gemv_f64.restype = ctypes.c_int
        _lib.q4_gemv_f64.argtypes = _lib.q4_gemv.argtypes
    return _lib


def dequant(raw: np.ndarray, ggml_type: int, rows: int, cols: int) -> np.ndarray:
    """Threaded block decode, bit-identical to ``oracle.q4_blocks.dequant``."""
    raw = np.ascontiguousarray(raw, np.uint8).reshape(-1)
    be, bb = {2: (32, 18), 12: (256, 144), 8: (32, 34), 6: (32, 22)}[ggml_type]
    nb = rows * cols // be
    assert raw.size == nb * bb
    out = np.empty(rows * cols, np.float32)
    rc = lib().q4_dequant(raw.ctypes.data, ggml_type, nb, out.ctypes.data)
    if rc:
        raise ValueError("unsupported ggml type")
    return out.reshape(rows, cols)


def gemv(raw: np.ndarray, ggml_type: int, N: int, K: int, x: np.ndarray) -> np.ndarray:
    raw = np.ascontiguousarray(raw, np.uint8).reshape(-1)
    x = np.ascontiguousarray(x, np.float32).reshape(-1, K)
    y = np.empty((x.shape[0], N), np.float32)
    rc = lib().q4_gemv(raw.ctypes.data, ggml_type, N, K, x.ctypes.data, x.shape[0], y.ctypes.data)
    if rc:
        raise ValueError(f"q4_gemv failed ({rc})")
    return y


def gemv_f64(raw: np.ndarray, ggml_type: int, N: int, K: int, x: np.ndarray) -> np.ndarray:
    """Same product with double-precision terms and sums (float64 ``[B, N]``)."""
    raw = np.ascontiguousarray(raw, np.uint8).reshape(-1)
    x = np.ascontiguousarray(x, np.float32).reshape(-1, K)
    y = np.empty((x.shape[0], N), np.float64)
    rc = lib().q4_gemv_f64(raw.ctypes.data, ggml_type, N, K, x.ctypes.data, x.shape[0], y.ctypes.data)
    if rc:
        raise ValueError(f"q4_gemv_f64 failed ({rc})")
    return y
