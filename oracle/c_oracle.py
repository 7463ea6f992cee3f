"""ctypes access to ``oracle/_build/liboracle_mx.so`` (the C restatement in ``mxquant.c``).  TEST INFRASTRUCTURE."""

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "liboracle_mx.so")
_lib = None


def build():
    subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = ctypes.CDLL(_SO)
        _lib.oracle_quantize_mx.argtypes = [
            ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
            ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
        ]
        _lib.oracle_quantize_mx.restype = None
    return _lib


def quantize_mx(x, threads=1):
    """``x``: numpy ``[M, K]`` float32, or uint16 holding bf16 bit patterns.  Returns ``(codes, scales)`` uint8."""
    x = np.ascontiguousarray(x)
    m, k = x.shape
    q = np.empty((m, k), dtype=np.uint8)
    s = np.empty((m, k // 32), dtype=np.uint8)
    lib().oracle_quantize_mx(x.ctypes.data, int(x.dtype != np.float32), m, k, k, q.ctypes.data, s.ctypes.data, threads)
    return q, s
