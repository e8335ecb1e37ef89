"""ctypes binding of the C ABI in include/sk_w2a8.h (lib/libsk_w2a8.so).

This is the stub a non-PyTorch host (or the parity tests) uses: plain pointers and sizes, one call per
entry point.  Loading fails loudly when the library has not been built; there is no fallback path.
"""
from __future__ import annotations

import ctypes
import os

from . import _build

SK_OK = 0
SK_ERR_NULL_POINTER = -1
SK_ERR_BAD_SHAPE = -2
SK_ERR_BAD_ALIGNMENT = -3
SK_ERR_UNSUPPORTED_ARCH = -4
SK_ERR_CUDA = -5
SK_ERR_DEVICE_TIMEOUT = -6
SK_ERR_BAD_ARGUMENT = -7
SK_ERR_OUT_OF_MEMORY = -8
SK_ERR_UNAVAILABLE = -9
SK_ERR_STATIC_SCRATCH_TOO_SMALL = -10

SK_OUT_F16, SK_OUT_BF16 = 0, 1
SK_WEIGHT_ROWMAJOR, SK_WEIGHT_TILED = 0, 1
SK_OPT_KERNEL, SK_OPT_TOKEN_TILE, SK_OPT_SPLIT_K, SK_OPT_PERSISTENT, SK_OPT_DEPENDENT_LAUNCH, SK_OPT_TMA_STORE = 1, 2, 3, 4, 5, 6
SK_OPT_WAIT_LIMIT_CYCLES, SK_OPT_TEST_SKIP_COPY, SK_OPT_STREAM_CTAS = 7, 8, 9
KERNEL_AUTO, KERNEL_TCGEN05, KERNEL_CUDA_CORE, KERNEL_TCGEN05_DECODE, KERNEL_TCGEN05_PAIR, KERNEL_TCGEN05_DECODE_BALANCED = 0, 1, 2, 3, 4, 5

_i64, _int, _vp = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p

# symbol -> (restype, argtypes); must list every function include/sk_w2a8.h declares
SIGNATURES = {
    "sk_w2a8_tiled_bytes": (_i64, [_i64, _i64]),
    "sk_w2a8_repack": (_int, [_vp, _i64, _i64, _vp, _vp]),
    "sk_w2a8_unrepack": (_int, [_vp, _i64, _i64, _vp, _vp]),
    "sk_w2a8_plan_create": (_int, [ctypes.POINTER(_vp), _int, _i64, _i64, _int, _int, _vp, _int, _vp, _int]),
    "sk_w2a8_plan_destroy": (_int, [_vp]),
    "sk_w2a8_set_option": (_int, [_vp, _int, _i64]),
    "sk_w2a8_plan_info": (_int, [_vp, ctypes.POINTER(_i64), ctypes.POINTER(_i64), ctypes.POINTER(_int),
                                 ctypes.POINTER(_int), ctypes.POINTER(_int), ctypes.POINTER(_int)]),
    "sk_w2a8_gemm": (_int, [_vp, _i64, _vp, _i64, _vp, _vp, _i64, _vp]),
    "sk_w2a8_gemm_scatter": (_int, [_vp, _i64, _vp, _i64, _vp, ctypes.POINTER(_vp), _int, _i64, _i64, _vp]),
    "sk_w2a8_gemm_rowscatter": (_int, [_vp, _i64, _vp, _i64, _vp, ctypes.POINTER(_vp), _int, _i64, _i64, _i64, _vp]),
    "sk_w2a8_gemm_debug_partials": (_int, [_vp, _i64, _vp, _i64, _vp, _vp]),
    "sk_quantize_activation_int8": (_int, [_vp, _i64, _i64, _i64, _vp, _i64, _vp, _vp]),
    "sk_silu_mul_quantize_int8": (_int, [_vp, _i64, _i64, _i64, _vp, _i64, _vp, _vp]),
    "sk_w2a8_debug_expander_image": (_int, [_vp, _int, _vp, _vp, _vp, _vp, _vp, _vp]),
    "sk_w2a8_debug_stream_cut": (_int, [_i64, _int, _int, _i64, ctypes.POINTER(_i64), ctypes.POINTER(_i64), ctypes.POINTER(_int)]),
    "sk_sum_row_blocks": (_int, [_vp, _int, _i64, _i64, _i64, _i64, _vp, _i64, _int, _vp]),
    "sk_w2a8_quantize_weight": (_int, [_vp, _i64, _i64, _i64, _int, _vp, _vp, _vp, _vp]),
    "sk_w2a8_mlp_workspace_bytes": (_i64, [_vp, _vp, _i64]),
    "sk_w2a8_mlp_forward": (_int, [_vp, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp]),
    "sk_w2a8_mlp_static_scratch_bytes": (_i64, []),
    "sk_w2a8_mlp_forward_static": (_int, [_vp, _vp, _i64, _vp, _i64, _vp, _i64, _vp]),
    "sk_w2a8_last_device_status": (_int, [_vp, ctypes.POINTER(_int)]),
    "sk_w2a8_last_cuda_error": (_int, [_vp]),
    "sk_device_status_string": (ctypes.c_char_p, [_int]),
    "sk_w2a8_query_launch": (_int, [_vp, _i64, ctypes.POINTER(_int), ctypes.POINTER(_int), ctypes.POINTER(_int),
                                    ctypes.POINTER(_int)]),
    "sk_w2a8_launch_floor_probe": (_int, [_vp, _i64, _vp]),
    "sk_status_string": (ctypes.c_char_p, [_int]),
    "sk_w2a8_version": (_int, []),
}

_lib = None


class SkError(RuntimeError):
    def __init__(self, status: int, what: str):
        self.status = status
        super().__init__(f"{what}: {status_string(status)} ({status})")


def load(path: str | None = None) -> ctypes.CDLL:
    """Loads lib/libsk_w2a8.so and types every entry point.  Raises if the library or a symbol is missing."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    path = path or _build.CUDA_LIB
    if not os.path.exists(path):
        raise ImportError(f"{path} is not built; run `python -m slimkernels_b200._build` (needs nvcc, sm_100a)")
    lib = ctypes.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the symbol is not exported
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


def status_string(status: int) -> str:
    return load().sk_status_string(status).decode()


def check(status: int, what: str) -> None:
    if status != SK_OK:
        raise SkError(status, what)


class Plan:
    """RAII wrapper over sk_w2a8_plan for callers that hold raw device pointers (ints)."""

    def __init__(self, device: int, N: int, K: int, group_size: int, zero_point: int, w_ptr: int,
                 w_scale_ptr: int, out_dtype: int = SK_OUT_F16, w_layout: int = SK_WEIGHT_ROWMAJOR):
        self._h = _vp()
        self.N, self.K, self.group_size, self.zero_point = N, K, group_size, zero_point
        check(load().sk_w2a8_plan_create(ctypes.byref(self._h), device, N, K, group_size, zero_point, w_ptr,
                                         w_layout, w_scale_ptr, out_dtype), "sk_w2a8_plan_create")

    @property
    def handle(self):
        return self._h

    def set_option(self, key: int, value: int) -> None:
        check(load().sk_w2a8_set_option(self._h, key, value), "sk_w2a8_set_option")

    def gemm(self, M, x_q_ptr, ld_x, x_scale_ptr, out_ptr, ld_out, stream=0) -> None:
        check(load().sk_w2a8_gemm(self._h, M, x_q_ptr, ld_x, x_scale_ptr, out_ptr, ld_out, stream), "sk_w2a8_gemm")

    def partials(self, M, x_q_ptr, ld_x, partials_ptr, stream=0) -> None:
        check(load().sk_w2a8_gemm_debug_partials(self._h, M, x_q_ptr, ld_x, partials_ptr, stream),
              "sk_w2a8_gemm_debug_partials")

    def device_status_string(self, code: int) -> str:
        return load().sk_device_status_string(code).decode()

    def device_status(self) -> int:
        v = _int(0)
        rc = load().sk_w2a8_last_device_status(self._h, ctypes.byref(v))
        if rc not in (SK_OK, SK_ERR_DEVICE_TIMEOUT):
            raise SkError(rc, "sk_w2a8_last_device_status")
        return v.value

    def query_launch(self, M: int):
        t, s, c, k = _int(), _int(), _int(), _int()
        check(load().sk_w2a8_query_launch(self._h, M, ctypes.byref(t), ctypes.byref(s), ctypes.byref(c),
                                          ctypes.byref(k)), "sk_w2a8_query_launch")
        return {"token_tile": t.value, "split_k": s.value, "ctas": c.value, "kernel": k.value}

    def close(self) -> None:
        if self._h:
            load().sk_w2a8_plan_destroy(self._h)
            self._h = _vp()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
