"""ctypes loader for the plain-C oracle (oracle/w2a8_oracle.c).  TEST INFRASTRUCTURE only."""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libw2a8_oracle.so")
_lib = None


def build() -> str:
    """Compile oracle/w2a8_oracle.c with the Makefile beside it; returns the .so path."""
    subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def pack_matrix(codes: np.ndarray) -> np.ndarray:
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    r, c = codes.shape
    out = np.empty((r, c // 4), dtype=np.uint8)
    rc = lib().oracle_pack_matrix(_p(codes), ctypes.c_int64(r), ctypes.c_int64(c), _p(out))
    if rc != 0:
        raise ValueError(f"oracle_pack_matrix rc={rc}")
    return out


def unpack_matrix(packed: np.ndarray) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    r, c = packed.shape
    out = np.empty((r, c * 4), dtype=np.uint8)
    lib().oracle_unpack_matrix(_p(packed), ctypes.c_int64(r), ctypes.c_int64(c), _p(out))
    return out


def dequantize_from_uint2(codes, scales_f16, group_size, zero_point=1):
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    scales_f16 = np.ascontiguousarray(scales_f16, dtype=np.float16)
    r, c = codes.shape
    out = np.empty((r, c), dtype=np.float16)
    lib().oracle_dequantize_from_uint2(_p(codes), _p(scales_f16), ctypes.c_int64(r), ctypes.c_int64(c),
                                       ctypes.c_int(group_size), ctypes.c_int(zero_point), _p(out))
    return out


def quantize_to_uint2(matrix, group_size):
    matrix = np.ascontiguousarray(matrix, dtype=np.float64)
    r, c = matrix.shape
    codes = np.empty((r, c), dtype=np.uint8)
    scales = np.empty((r // group_size, c), dtype=np.float64)
    lib().oracle_quantize_to_uint2(_p(matrix), ctypes.c_int64(r), ctypes.c_int64(c),
                                   ctypes.c_int(group_size), _p(codes), _p(scales))
    return codes, scales


def w2a8_partials(x_q, w_packed, group_size=128, zero_point=1):
    x_q = np.ascontiguousarray(x_q, dtype=np.int8)
    w_packed = np.ascontiguousarray(w_packed, dtype=np.uint8)
    M, K = x_q.shape
    N = w_packed.shape[0]
    out = np.empty((K // group_size, M, N), dtype=np.int32)
    lib().oracle_w2a8_partials(_p(x_q), _p(w_packed), ctypes.c_int64(M), ctypes.c_int64(N),
                               ctypes.c_int64(K), ctypes.c_int(group_size), ctypes.c_int(zero_point),
                               _p(out))
    return out


def w2a8_gemm(x_q, x_scale, w_packed, w_scale_f16, group_size=128, zero_point=1):
    x_q = np.ascontiguousarray(x_q, dtype=np.int8)
    x_scale = np.ascontiguousarray(x_scale, dtype=np.float32)
    w_packed = np.ascontiguousarray(w_packed, dtype=np.uint8)
    w_scale_f16 = np.ascontiguousarray(w_scale_f16, dtype=np.float16)
    M, K = x_q.shape
    N = w_packed.shape[0]
    out = np.empty((M, N), dtype=np.float32)
    lib().oracle_w2a8_gemm(_p(x_q), _p(x_scale), _p(w_packed), _p(w_scale_f16), ctypes.c_int64(M),
                           ctypes.c_int64(N), ctypes.c_int64(K), ctypes.c_int(group_size),
                           ctypes.c_int(zero_point), _p(out))
    return out
