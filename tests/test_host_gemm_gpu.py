"""W2A8Plan.gemm_host: operands in pinned host memory, copies and GEMM chunks overlapped on three streams;
must give the bits of the plain device call."""
import numpy as np
import pytest
import torch

from gpu_util import random_problem

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _need_gpu(built_libs):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")


@pytest.mark.parametrize("M,chunk", [(300, 128), (1024, 512), (77, 512)])
def test_gemm_host_matches_device_call(M, chunk):
    from slimkernels_b200.torch import W2A8Plan
    x_q, xs, wp, ws = random_problem(M, 384, 512, 128, seed=M)
    plan = W2A8Plan(torch.from_numpy(wp).cuda(), torch.from_numpy(ws).cuda(), group_size=128)
    d_x, d_xs = torch.from_numpy(x_q).cuda(), torch.from_numpy(xs).cuda()
    # the same chunks through the plain device call (the token tile, hence the order of the fp32 sums, follows the
    # number of tokens in a call)
    want = torch.cat([plan.gemm(d_x[lo:lo + chunk], d_xs[lo:lo + chunk]) for lo in range(0, M, chunk)]).cpu()
    whole = plan.gemm(d_x, d_xs).cpu()
    assert (want.float() - whole.float()).abs().max().item() <= 1e-2
    h_x, h_xs = torch.from_numpy(x_q).pin_memory(), torch.from_numpy(xs).pin_memory()
    h_out = torch.full((M, 384), float("nan"), dtype=torch.float16).pin_memory()
    for _ in range(2):                                  # the second call reuses the staging buffers
        h_out.fill_(float("nan"))
        plan.gemm_host(h_x, h_xs, h_out, chunk_tokens=chunk)
        torch.cuda.synchronize()
        assert torch.equal(h_out, want)
    with pytest.raises(TypeError):
        plan.gemm_host(h_x.cuda(), h_xs, h_out)
    with pytest.raises(ValueError):
        plan.gemm_host(h_x, h_xs, h_out[:, :128])
