"""The C-ABI library: builds, loads, exports every symbol include/sk_w2a8.h declares, and rejects bad
arguments before touching the device.  No compute is launched here."""
import ctypes
import os
import re

import numpy as np
import pytest

from conftest import ROOT


def test_library_exports_every_declared_symbol(built_libs):
    from slimkernels_b200 import capi
    header = open(os.path.join(ROOT, "include", "sk_w2a8.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(sk_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations parsed"
    lib = capi.load()
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in sk_w2a8.h but not exported"
    assert declared == set(capi.SIGNATURES), "ctypes binding and header disagree"
    assert lib.sk_w2a8_version() >= 100


def test_status_strings(built_libs):
    from slimkernels_b200 import capi
    assert capi.status_string(capi.SK_OK) == "ok"
    for code in range(-10, 0):
        assert capi.status_string(code) not in ("", "unknown status")
    assert capi.status_string(-1234) == "unknown status"


def test_argument_validation_without_device(built_libs):
    from slimkernels_b200 import capi
    lib = capi.load()
    h = ctypes.c_void_p()
    fake = 4096  # never dereferenced: validation fails first
    create = lib.sk_w2a8_plan_create
    assert create(None, 0, 128, 128, 128, 1, fake, 0, fake, 0) == capi.SK_ERR_NULL_POINTER
    assert create(ctypes.byref(h), 0, 128, 128, 128, 1, None, 0, fake, 0) == capi.SK_ERR_NULL_POINTER
    assert create(ctypes.byref(h), 0, 0, 128, 128, 1, fake, 0, fake, 0) == capi.SK_ERR_BAD_SHAPE
    assert create(ctypes.byref(h), 0, 128, 100, 128, 1, fake, 0, fake, 0) == capi.SK_ERR_BAD_SHAPE   # K % G
    assert create(ctypes.byref(h), 0, 128, 192, 48, 1, fake, 0, fake, 0) == capi.SK_ERR_BAD_SHAPE    # G % 32
    assert create(ctypes.byref(h), 0, 128, 192, 96, 1, fake, 0, fake, 0) == capi.SK_ERR_BAD_SHAPE    # 96 vs 128
    assert create(ctypes.byref(h), 0, 128, 128, 128, 7, fake, 0, fake, 0) == capi.SK_ERR_BAD_ARGUMENT
    assert create(ctypes.byref(h), 0, 128, 128, 128, 1, fake, 5, fake, 0) == capi.SK_ERR_BAD_ARGUMENT
    assert create(ctypes.byref(h), 0, 128, 128, 128, 1, fake, 0, fake, 9) == capi.SK_ERR_BAD_ARGUMENT
    assert create(ctypes.byref(h), 0, 128, 128, 128, 1, fake + 1, 1, fake, 0) == capi.SK_ERR_BAD_ALIGNMENT
    assert not h.value
    assert lib.sk_w2a8_plan_destroy(None) == capi.SK_ERR_NULL_POINTER
    assert lib.sk_w2a8_gemm(None, 1, fake, 128, fake, fake, 128, None) == capi.SK_ERR_NULL_POINTER
    assert lib.sk_w2a8_gemm_debug_partials(None, 1, fake, 128, None, None) == capi.SK_ERR_NULL_POINTER
    assert lib.sk_w2a8_repack(None, 128, 128, fake, None) == capi.SK_ERR_NULL_POINTER
    assert lib.sk_w2a8_repack(fake, 128, 100, fake, None) == capi.SK_ERR_BAD_SHAPE
    assert lib.sk_w2a8_tiled_bytes(4096, 4096) == 4096 * 4096 // 4
    assert lib.sk_w2a8_tiled_bytes(130, 160) == 2 * 2 * 4096


def test_torch_extension_registers_ops(built_libs):
    import torch
    from slimkernels_b200.torch import ops
    ops.load_extension()
    for name in ("w2a8_plan_create", "w2a8_plan_gemm", "w2a8_plan_gemm_out", "w2a8_plan_partials",
                 "w2a8_repack", "w2a8_unrepack"):
        assert hasattr(torch.ops.slimkernels, name)


@pytest.mark.skipif(__import__("torch").cuda.is_available(), reason="checks the no-GPU failure mode")
def test_product_path_fails_loudly_without_gpu(built_libs):
    import torch
    from slimkernels_b200.torch import ops
    x_q = torch.zeros(4, 128, dtype=torch.int8)
    xs = torch.ones(4)
    wp = torch.zeros(128, 32, dtype=torch.uint8)
    ws = torch.ones(1, 128, dtype=torch.float16)
    with pytest.raises(RuntimeError):
        ops.w2a8_gemm(x_q, xs, wp, ws)


def test_balanced_split_cut_is_a_partition_and_owner_inverts_it():
    """Host arithmetic of the balanced-split decode kernel: the CTA ranges tile [0, units) without gaps, differ by at
    most one half stage, and stream_owner names the range that holds a half stage (the kernel derives the slots of a
    shared tile from it)."""
    import ctypes
    from slimkernels_b200 import capi
    lib = capi.load()
    rng = np.random.default_rng(0)
    cases = [(1, 1), (16, 16), (1536, 296), (5504, 296), (5504, 148), (14336, 296), (7, 3), (1000, 999)]
    cases += [(int(u), int(c)) for u in rng.integers(1, 5000, size=20) for c in rng.integers(1, 400, size=2) if c <= u]
    for units, ctas in cases:
        b, e, o = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int()
        prev_end, sizes = 0, []
        for c in range(ctas):
            assert lib.sk_w2a8_debug_stream_cut(units, ctas, c, 0, ctypes.byref(b), ctypes.byref(e), None) == capi.SK_OK
            assert b.value == prev_end and e.value >= b.value
            sizes.append(e.value - b.value)
            prev_end = e.value
            for x in {b.value, e.value - 1, (b.value + e.value) // 2}:
                if b.value <= x < e.value:
                    assert lib.sk_w2a8_debug_stream_cut(units, ctas, 0, x, None, None, ctypes.byref(o)) == capi.SK_OK
                    assert o.value == c, (units, ctas, c, x, o.value)
        assert prev_end == units and max(sizes) - min(sizes) <= 1 and min(sizes) >= 1
    assert lib.sk_w2a8_debug_stream_cut(4, 5, 0, 0, None, None, None) == capi.SK_ERR_BAD_ARGUMENT
