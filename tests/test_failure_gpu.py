"""Failure behaviour on the device, in the form that cannot hurt a GPU: every wait inside the kernels has a limit,
after which the kernel RETURNS and leaves a status word for the host.  Here the limit is made short and the producer
is told to leave out one pipeline stage's copies (a test hook of the library), so the waits for that stage run out.
Nothing traps, faults or spins without a limit; the context stays usable and the next ordinary call is correct.

The reference's counterpart is abort-style error macros (slimkernels/cute/gemm/wgmma_sm90_W2A8.cu:489-505) and
unbounded barrier waits (:356, :381)."""
import numpy as np
import pytest
import torch

from oracle import w2a8_oracle as O
from slimkernels_b200 import capi

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _need_gpu(built_libs):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests selected but no CUDA device is visible")


from gpu_util import DeviceProblem, random_problem, to_np  # noqa: E402

# role * 16 + barrier kind: the roles that wait for the copies of a stage
# Every role of the CTA ends up waiting on the missing copies, directly or through the role before it, with the same
# limit and from about the same moment: whichever notices first names the stall.  All of these are consequences of
# the one copy that never came.
WAITS_FOR_COPIES = {0x21: "expander", 0x31: "MMA issuer", 0x11: "producer", 0x22: "expander", 0x32: "MMA issuer",
                    0x33: "MMA issuer", 0x41: "epilogue"}


@pytest.mark.parametrize("kernel,M,skip", [
    (capi.KERNEL_TCGEN05, 40, 2),             # general kernel, 64-token tile: K block 1 of 8 never arrives
    (capi.KERNEL_TCGEN05, 300, 1),            # 256-token tile, two token tiles, first K block
    (capi.KERNEL_TCGEN05_PAIR, 300, 3),       # pairs of CTAs (cta_group::2): both CTAs of every pair give up and leave
    (capi.KERNEL_TCGEN05_DECODE, 16, 1),      # decode kernel: the first load stage (K blocks 0..3)
    (capi.KERNEL_TCGEN05_DECODE, 16, 5),      # decode kernel: the second load stage
    (capi.KERNEL_TCGEN05_DECODE_BALANCED, 16, 1),   # balanced-split decode kernel: the first load stage of every CTA;
                                                    # the counters of half-counted tiles are cleared with the status
])
def test_wait_limit_expires_kernel_returns_and_next_call_is_correct(kernel, M, skip):
    x_q, xs, wp, ws = random_problem(M, 256, 1024, 128, seed=M + skip)
    dp = DeviceProblem(x_q, xs, wp, ws).force(kernel=kernel, split_k=1)
    y_ref = O.w2a8_gemm_dequant_path(x_q, xs, wp, ws)
    assert np.abs(to_np(dp.gemm()) - y_ref).max() <= 1e-2          # healthy first

    dp.plan.set_option(capi.SK_OPT_WAIT_LIMIT_CYCLES, 200000)      # ~0.1 ms instead of ~0.5 s
    dp.plan.set_option(capi.SK_OPT_TEST_SKIP_COPY, skip)
    out = torch.zeros(M, 256, dtype=torch.float16, device="cuda")
    lib = capi.load()
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.sk_w2a8_gemm(dp.plan.handle, M, dp.x_q.data_ptr(), 1024, dp.x_scale.data_ptr(), out.data_ptr(), 256, stream)
    assert rc == capi.SK_OK                                        # the launch itself is fine
    torch.cuda.synchronize()                                       # ... and the kernel comes back by itself
    code = capi._int(0)
    rc = lib.sk_w2a8_last_device_status(dp.plan.handle, code)
    assert rc == capi.SK_ERR_DEVICE_TIMEOUT
    assert code.value in WAITS_FOR_COPIES, hex(code.value)
    text = dp.plan.device_status_string(code.value)
    assert text != "unknown device status" and WAITS_FOR_COPIES[code.value].split()[0].lower() in text.lower()
    assert "expired" in capi.status_string(rc)
    # reading the status cleared it
    assert dp.plan.device_status() == 0

    # the same plan, hook off: bit-identical to the healthy result, and the context is intact
    dp.plan.set_option(capi.SK_OPT_TEST_SKIP_COPY, 0)
    dp.plan.set_option(capi.SK_OPT_WAIT_LIMIT_CYCLES, 0)
    y_a, y_b = dp.gemm(), dp.gemm()
    assert torch.equal(y_a, y_b)
    assert np.abs(to_np(y_a) - y_ref).max() <= 1e-2
    np.testing.assert_array_equal(to_np(dp.partials()), O.w2a8_partials(x_q, wp, 128))


def test_wait_limit_option_validation():
    x_q, xs, wp, ws = random_problem(4, 128, 256, 128, seed=1)
    dp = DeviceProblem(x_q, xs, wp, ws)
    with pytest.raises(capi.SkError):
        dp.plan.set_option(capi.SK_OPT_WAIT_LIMIT_CYCLES, 10)      # below the floor of 1000 cycles
    with pytest.raises(capi.SkError):
        dp.plan.set_option(capi.SK_OPT_WAIT_LIMIT_CYCLES, -1)
    dp.plan.set_option(capi.SK_OPT_WAIT_LIMIT_CYCLES, 0)
    assert capi.load().sk_device_status_string(0).decode() == "no wait expired"
    assert "unknown" in capi.load().sk_device_status_string(0x7777).decode()
