"""The allocation-free MLP entry point, sk_w2a8_mlp_forward_static.

Who needs it: a host that has given all device memory away at start-up (a serving process with its own arena, an
embedded or real-time runtime with a fixed memory budget) cannot call cudaMalloc any more, and cannot let a
framework do it on its behalf, yet the ordinary MLP entry point wants a workspace for its intermediates.  The
static variant keeps those intermediates in a fixed array inside the library image instead.

This file is collected last on purpose (its name sorts after every other test file), so that a run that stops at
the first failure has already run everything else.  It must hold both alone in a fresh process and after the rest
of the suite: it only uses the C ABI through ctypes and its own buffers.

Checked here, on two calls in a row with different inputs (the array is shared and keeps the previous call's
contents): the static entry point produces exactly the bytes of the workspace entry point (same four kernels, so
the tolerance is zero), it refuses a problem larger than its buffer before launching anything, and the call in
between did not disturb the result of the next one.
"""
import numpy as np
import pytest
import torch

from slimkernels_b200 import capi

pytestmark = pytest.mark.gpu


def _problem(M, hidden, inter, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((M, hidden)).astype(np.float16)
    gu_p = rng.integers(0, 256, size=(2 * inter, hidden // 4), dtype=np.uint8)
    gu_s = rng.uniform(0.001, 0.01, size=(hidden // 128, 2 * inter)).astype(np.float16)
    dn_p = rng.integers(0, 256, size=(hidden, inter // 4), dtype=np.uint8)
    dn_s = rng.uniform(0.001, 0.01, size=(inter // 128, hidden)).astype(np.float16)
    return x, gu_p, gu_s, dn_p, dn_s


def test_static_mlp_matches_workspace_mlp_twice_in_a_row(built_libs):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests selected but no CUDA device is visible")
    lib = capi.load()
    dev = torch.device("cuda:0")
    hidden, inter = 1024, 2816
    assert lib.sk_w2a8_mlp_static_scratch_bytes() == 8 << 20
    _, gu_p, gu_s, dn_p, dn_s = _problem(1, hidden, inter, seed=11)
    t = [torch.from_numpy(a).to(dev) for a in (gu_p, gu_s, dn_p, dn_s)]
    gu = capi.Plan(0, 2 * inter, hidden, 128, 1, t[0].data_ptr(), t[1].data_ptr())
    dn = capi.Plan(0, hidden, inter, 128, 1, t[2].data_ptr(), t[3].data_ptr())
    stream = torch.cuda.current_stream(dev).cuda_stream

    # every buffer of the test exists before the entry point under test is called
    cases = []
    for M, seed in [(24, 1), (7, 2)]:            # second call: fewer rows than the first left behind in the array
        x = torch.from_numpy(_problem(M, hidden, inter, seed)[0]).to(dev)
        nbytes = lib.sk_w2a8_mlp_workspace_bytes(gu.handle, dn.handle, M)
        assert 0 < nbytes <= 8 << 20
        cases.append((M, x, torch.empty(nbytes, dtype=torch.uint8, device=dev),
                      torch.zeros(M, hidden, dtype=torch.float16, device=dev),
                      torch.zeros(M, hidden, dtype=torch.float16, device=dev)))
    torch.cuda.synchronize(dev)

    for M, x, ws, out_ref, out_static in cases:           # the reference results first: this also loads every kernel
        rc = lib.sk_w2a8_mlp_forward(gu.handle, dn.handle, M, x.data_ptr(), hidden, out_ref.data_ptr(), hidden,
                                     ws.data_ptr(), ws.numel(), stream)
        assert rc == capi.SK_OK
    torch.cuda.synchronize(dev)
    free = []
    for M, x, ws, out_ref, out_static in cases:
        rc = lib.sk_w2a8_mlp_forward_static(gu.handle, dn.handle, M, x.data_ptr(), hidden, out_static.data_ptr(),
                                            hidden, stream)
        assert rc == capi.SK_OK, capi.status_string(rc)
        torch.cuda.synchronize(dev)
        free.append(torch.cuda.mem_get_info(dev)[0])
    # the first call looked the array's address up; the second call must not take any device memory
    assert free[1] >= free[0], "the allocation-free entry point consumed device memory"
    assert gu.device_status() == 0 and dn.device_status() == 0
    for M, x, ws, out_ref, out_static in cases:
        assert torch.isfinite(out_ref).all() and out_ref.abs().max() > 0
        assert torch.equal(out_static, out_ref), f"M={M}: static and workspace variants differ"


def test_static_mlp_refuses_what_does_not_fit(built_libs):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests selected but no CUDA device is visible")
    lib = capi.load()
    dev = torch.device("cuda:0")
    hidden, inter = 1024, 2816
    _, gu_p, gu_s, dn_p, dn_s = _problem(1, hidden, inter, seed=11)
    t = [torch.from_numpy(a).to(dev) for a in (gu_p, gu_s, dn_p, dn_s)]
    gu = capi.Plan(0, 2 * inter, hidden, 128, 1, t[0].data_ptr(), t[1].data_ptr())
    dn = capi.Plan(0, hidden, inter, 128, 1, t[2].data_ptr(), t[3].data_ptr())
    M = 1024                                           # needs about 15 MB of intermediates
    assert lib.sk_w2a8_mlp_workspace_bytes(gu.handle, dn.handle, M) > 8 << 20
    x = torch.zeros(M, hidden, dtype=torch.float16, device=dev)
    out = torch.full((M, hidden), 7.0, dtype=torch.float16, device=dev)
    rc = lib.sk_w2a8_mlp_forward_static(gu.handle, dn.handle, M, x.data_ptr(), hidden, out.data_ptr(), hidden,
                                        torch.cuda.current_stream(dev).cuda_stream)
    assert rc == capi.SK_ERR_STATIC_SCRATCH_TOO_SMALL
    assert "scratch" in capi.status_string(rc)
    torch.cuda.synchronize(dev)
    assert bool((out == 7.0).all()), "a refused call must not launch anything"
    assert lib.sk_w2a8_mlp_forward_static(gu.handle, dn.handle, 4, None, hidden, out.data_ptr(), hidden, None) \
        == capi.SK_ERR_NULL_POINTER
