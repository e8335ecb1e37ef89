"""The registered op torch.ops.slimkernels.w2a8_gemm (call shape of the reference's notebook wrapper
wint2_gemm(activation, weight, scale) -> out, triton.ipynb:235-270) and the plan caches behind it."""
import gc

import numpy as np
import pytest
import torch

from oracle import w2a8_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _need_gpu(built_libs):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests selected but no CUDA device is visible")
    from slimkernels_b200.torch import load_extension
    load_extension()


from gpu_util import random_problem  # noqa: E402


def _dev(*arrays):
    return [torch.from_numpy(a).cuda() for a in arrays]


def test_registered_op_matches_oracle_and_defaults():
    x_q, xs, wp, ws = random_problem(37, 384, 1024, 128, seed=2)
    d = _dev(x_q, xs, wp, ws)
    y = torch.ops.slimkernels.w2a8_gemm(*d)                      # group_size=128, zero_point=1, float16
    assert y.dtype == torch.float16 and tuple(y.shape) == (37, 384)
    assert np.abs(y.float().cpu().numpy() - O.w2a8_gemm_dequant_path(x_q, xs, wp, ws)).max() <= 1e-2
    y2 = torch.ops.slimkernels.w2a8_gemm(*d, 128, 2, torch.bfloat16)
    assert y2.dtype == torch.bfloat16
    ref2 = O.w2a8_gemm_dequant_path(x_q, xs, wp, ws, 128, 2)
    assert np.abs(y2.float().cpu().numpy() - ref2).max() <= 1e-2 + np.abs(ref2).max() * 2.0 ** -8
    p = torch.ops.slimkernels.w2a8_partials(d[0], d[2], d[3])
    np.testing.assert_array_equal(p.cpu().numpy(), O.w2a8_partials(x_q, wp, 128))
    with pytest.raises(RuntimeError):
        torch.ops.slimkernels.w2a8_gemm(d[0], d[1], d[2], d[3], 128, 1, torch.float32)


def test_plan_cache_follows_the_weight_tensor():
    """One plan per live weight tensor: reused across calls, rebuilt after an in-place write, dropped with the tensor."""
    x_q, xs, wp, ws = random_problem(8, 256, 512, 128, seed=3)
    d_x, d_xs, d_wp, d_ws = _dev(x_q, xs, wp, ws)
    count = torch.ops.slimkernels.w2a8_cached_plan_count
    base = count()
    y0 = torch.ops.slimkernels.w2a8_gemm(d_x, d_xs, d_wp, d_ws)
    assert count() == base + 1
    assert torch.equal(torch.ops.slimkernels.w2a8_gemm(d_x, d_xs, d_wp, d_ws), y0)
    assert count() == base + 1
    wp2 = np.random.default_rng(4).integers(0, 256, size=wp.shape, dtype=np.uint8)
    d_wp.copy_(torch.from_numpy(wp2).cuda())                     # in-place: same tensor, new contents
    y1 = torch.ops.slimkernels.w2a8_gemm(d_x, d_xs, d_wp, d_ws)
    assert count() == base + 1
    assert np.abs(y1.float().cpu().numpy() - O.w2a8_gemm_dequant_path(x_q, xs, wp2, ws)).max() <= 1e-2
    torch.cuda.synchronize()
    del d_wp, y0, y1
    gc.collect()
    assert count() == base                                       # the cache held the weight only weakly


def test_linear_module_rebuilds_its_plan_when_the_buffers_change():
    from slimkernels_b200.torch import W2A8Linear
    x_q, xs, wp, ws = random_problem(5, 256, 512, 128, seed=6)
    lin = W2A8Linear(*_dev(wp, ws))
    d_x, d_xs = _dev(x_q, xs)
    y0 = lin.forward_quantized(d_x, d_xs)
    assert np.abs(y0.float().cpu().numpy() - O.w2a8_gemm_dequant_path(x_q, xs, wp, ws)).max() <= 1e-2
    wp2 = np.random.default_rng(7).integers(0, 256, size=wp.shape, dtype=np.uint8)
    lin.load_state_dict({"w_packed": torch.from_numpy(wp2), "w_scale": torch.from_numpy(ws)})
    y1 = lin.forward_quantized(d_x, d_xs)
    assert np.abs(y1.float().cpu().numpy() - O.w2a8_gemm_dequant_path(x_q, xs, wp2, ws)).max() <= 1e-2


def test_gemm_out_checks_dtype_and_width_against_the_plan():
    from slimkernels_b200.torch import W2A8Plan
    x_q, xs, wp, ws = random_problem(4, 256, 512, 128, seed=8)
    d_x, d_xs, d_wp, d_ws = _dev(x_q, xs, wp, ws)
    plan = W2A8Plan(d_wp, d_ws, out_dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        plan.gemm(d_x, d_xs, out=torch.empty(4, 256, dtype=torch.float16, device="cuda"))
    with pytest.raises(RuntimeError):
        plan.gemm(d_x, d_xs, out=torch.empty(4, 128, dtype=torch.bfloat16, device="cuda"))
    plan.gemm(d_x, d_xs, out=torch.empty(4, 256, dtype=torch.bfloat16, device="cuda"))
    assert plan.query_launch(4)["kernel"] == 3


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_mlp_forward_runs_on_the_plans_device_whatever_is_current():
    from slimkernels_b200 import capi
    lib = capi.load()
    hidden, inter, M = 256, 384, 8
    rng = np.random.default_rng(5)
    x = rng.standard_normal((M, hidden)).astype(np.float16)
    gu_p = rng.integers(0, 256, size=(2 * inter, hidden // 4), dtype=np.uint8)
    gu_s = rng.uniform(0.001, 0.01, size=(hidden // 128, 2 * inter)).astype(np.float16)
    dn_p = rng.integers(0, 256, size=(hidden, inter // 4), dtype=np.uint8)
    dn_s = rng.uniform(0.001, 0.01, size=(inter // 128, hidden)).astype(np.float16)
    dev = torch.device("cuda:1")
    t = [torch.from_numpy(a).to(dev) for a in (gu_p, gu_s, dn_p, dn_s)]
    gu = capi.Plan(1, 2 * inter, hidden, 128, 1, t[0].data_ptr(), t[1].data_ptr())
    dn = capi.Plan(1, hidden, inter, 128, 1, t[2].data_ptr(), t[3].data_ptr())
    nbytes = lib.sk_w2a8_mlp_workspace_bytes(gu.handle, dn.handle, M)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    d_x = torch.from_numpy(x).to(dev)
    out = torch.empty(M, hidden, dtype=torch.float16, device=dev)
    torch.cuda.synchronize(dev)
    torch.cuda.set_device(0)                                      # another device is current for the calling thread
    assert lib.sk_w2a8_mlp_forward(gu.handle, dn.handle, M, d_x.data_ptr(), hidden, out.data_ptr(), hidden,
                                   ws.data_ptr(), nbytes, None) == 0
    assert torch.cuda.current_device() == 0
    torch.cuda.synchronize(dev)
    y_ref = O.llama_mlp(x, gu_p, gu_s, dn_p, dn_s, 128)
    assert np.abs(out.float().cpu().numpy() - y_ref).max() <= 1e-2 * np.abs(y_ref).max() + 1e-2


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_sum_row_blocks_adds_in_block_order_in_fp32(dtype):
    """The add half of the reduce-scatter: fp32 sum of the row blocks in index order, rounded once (bit-exact against
    the same sum spelled out in torch)."""
    from slimkernels_b200.torch import load_extension
    load_extension()
    g = torch.Generator(device="cuda").manual_seed(3)
    blocks = (torch.randn(5, 300, 264, device="cuda", generator=g) * 3).to(dtype)
    acc = blocks[0].float()
    for b in range(1, 5):
        acc = acc + blocks[b].float()
    out = torch.ops.slimkernels.sum_row_blocks(blocks)
    assert out.dtype == dtype and torch.equal(out, acc.to(dtype))
    assert torch.equal(torch.ops.slimkernels.sum_row_blocks(blocks[:1]), blocks[0])
    with pytest.raises(RuntimeError):
        torch.ops.slimkernels.sum_row_blocks(blocks[:, :, :260])          # not contiguous
    with pytest.raises(RuntimeError):
        torch.ops.slimkernels.sum_row_blocks(blocks[:, :, :4].contiguous())   # N % 8 != 0
