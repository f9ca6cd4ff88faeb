"""ctypes binding of the C restatement (oracle/libtfp8_oracle.so) and, when it was built, of the
shim around the reference's own fp8.h (oracle/_ref/libref_fp8h.so).

TEST INFRASTRUCTURE ONLY -- see tfp8_oracle.py. Used by the tests (cross-check of the numpy
oracle) and by the benchmark's CPU-baseline leg (it is what gets timed on the host cores)."""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_P, _L, _I = ctypes.c_void_p, ctypes.c_long, ctypes.c_int


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def load():
    lib = ctypes.CDLL(os.path.join(_HERE, "libtfp8_oracle.so"))
    lib.oracle_decode_table.argtypes = [_I, _P]
    lib.oracle_encode.argtypes = [_P, _P, _L, _I, _I]
    lib.oracle_dequantize.argtypes = [_P, _P, _P, _L, _L, _L, _I]
    lib.oracle_matmul.argtypes = [_P, _P, _P, _P, _L, _L, _L]
    lib.oracle_linear_forward.argtypes = [_P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _I]
    return lib


def load_ref():
    """The reference's fp8.h behind C entry points, or None if it was not built."""
    path = os.path.join(_HERE, "_ref", "libref_fp8h.so")
    if not os.path.exists(path):
        return None
    lib = ctypes.CDLL(path)
    lib.ref_fp8_decode.argtypes, lib.ref_fp8_decode.restype = [ctypes.c_ubyte, _I], ctypes.c_float
    lib.ref_fp8_encode.argtypes, lib.ref_fp8_encode.restype = [ctypes.c_float, _I], ctypes.c_ubyte
    lib.ref_fp8_build_lut.argtypes = [_I, _P]
    return lib


FMT_ID = {"e4m3fn": 0, "e5m2": 1}


def decode_table(fmt):
    out = np.empty(256, np.float32)
    load().oracle_decode_table(FMT_ID[fmt], _ptr(out))
    return out


def encode(x, fmt, nan_mode="cast"):
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(x.shape, np.uint8)
    load().oracle_encode(_ptr(x), _ptr(out), x.size, FMT_ID[fmt], int(nan_mode == "canonical"))
    return out


def linear_forward(x, q, s, bias, fmt, group_size, work=None, lib=None):
    """float32 y = x @ (table[q] * s).T + bias, dequantize-then-matmul on all host threads."""
    lib = lib or load()
    x = np.ascontiguousarray(x, np.float32)
    q = np.ascontiguousarray(q, np.uint8)
    s = np.ascontiguousarray(s, np.float32)
    M, K = x.shape
    N = q.shape[0]
    if work is None:
        work = np.empty((N, K), np.float32)
    y = np.empty((M, N), np.float32)
    b = np.ascontiguousarray(bias, np.float32) if bias is not None else None
    lib.oracle_linear_forward(_ptr(x), _ptr(q), _ptr(s), _ptr(b), _ptr(work), _ptr(y), M, N, K, group_size, FMT_ID[fmt])
    return y
