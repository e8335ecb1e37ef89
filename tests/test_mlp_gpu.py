"""Activation quantiser, SiLU*up re-quantiser and the W2A8 Llama MLP block (benchmark config 4) against the oracle."""
import ctypes

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


@pytest.mark.parametrize("M,K", [(1, 4096), (16, 4096), (7, 11008), (33, 128), (5, 28672), (3, 8)])
def test_quantize_activation_bit_exact(M, K):
    rng = np.random.default_rng(M * 7 + K)
    x = rng.standard_normal((M, K)).astype(np.float16)
    if M > 2:
        x[1] = 0          # an all-zero row: scale 1.0, codes 0
        x[2, :8] = [65504, -65504, 0.5, -0.5, 1.5, 2.5, -1.5, -2.5]   # range ends and rounding ties
    lib = capi.load()
    d_x = torch.from_numpy(x).cuda()
    d_q = torch.full((M, K), 99, dtype=torch.int8, device="cuda")
    d_s = torch.zeros(M, dtype=torch.float32, device="cuda")
    rc = lib.sk_quantize_activation_int8(d_x.data_ptr(), K, M, K, d_q.data_ptr(), K, d_s.data_ptr(),
                                         torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    q_ref, s_ref = O.quantize_activation_int8(x)
    np.testing.assert_array_equal(d_s.cpu().numpy(), s_ref)
    np.testing.assert_array_equal(d_q.cpu().numpy(), q_ref)


@pytest.mark.parametrize("M,I", [(1, 11008), (16, 11008), (9, 128), (4, 28672), (3, 6144), (3, 6152), (2, 60000)])
def test_silu_mul_quantize(M, I):
    rng = np.random.default_rng(M + I)
    gu = (rng.standard_normal((M, 2 * I)) * 3).astype(np.float16)
    lib = capi.load()
    d_gu = torch.from_numpy(gu).cuda()
    d_q = torch.zeros((M, I), dtype=torch.int8, device="cuda")
    d_s = torch.zeros(M, dtype=torch.float32, device="cuda")
    rc = lib.sk_silu_mul_quantize_int8(d_gu.data_ptr(), 2 * I, M, I, d_q.data_ptr(), I, d_s.data_ptr(),
                                       torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    g, u = gu[:, :I].astype(np.float32), gu[:, I:].astype(np.float32)
    h = (g / (np.float32(1.0) + np.exp(-g))) * u
    q_ref, s_ref = O.quantize_activation_int8(h)
    # expf differs from numpy's exp by an ulp here and there: scales agree to 1e-6 relative, codes to one step
    np.testing.assert_allclose(d_s.cpu().numpy(), s_ref, rtol=2e-6)
    diff = np.abs(d_q.cpu().numpy().astype(np.int32) - q_ref.astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() < 2e-3


def _mlp_problem(M, hidden, inter, seed=0):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((M, hidden)).astype(np.float16)
    gu_p = rng.integers(0, 256, size=(2 * inter, hidden // 4), dtype=np.uint8)
    gu_s = rng.uniform(0.001, 0.01, size=(hidden // 128, 2 * inter)).astype(np.float16)
    dn_p = rng.integers(0, 256, size=(hidden, inter // 4), dtype=np.uint8)
    dn_s = rng.uniform(0.001, 0.01, size=(inter // 128, hidden)).astype(np.float16)
    return x, gu_p, gu_s, dn_p, dn_s


@pytest.mark.parametrize("M", [1, 16, 512])
def test_llama_mlp_block_against_oracle(M):
    """Llama-2-7B MLP: hidden 4096, intermediate 11008 (config 4).  Tolerance: 1e-2 of the output's max magnitude
    (a one-step difference of an int8 activation code moves an output by about s_act * s_w * |x| ~ 1e-3 of it)."""
    from slimkernels_b200.torch import W2A8Linear, W2A8LlamaMLP
    hidden, inter = 4096, 11008
    x, gu_p, gu_s, dn_p, dn_s = _mlp_problem(M, hidden, inter, seed=M)
    dev = torch.device("cuda:0")
    mlp = W2A8LlamaMLP(W2A8Linear(torch.from_numpy(gu_p).to(dev), torch.from_numpy(gu_s).to(dev)),
                       W2A8Linear(torch.from_numpy(dn_p).to(dev), torch.from_numpy(dn_s).to(dev)))
    y = mlp(torch.from_numpy(x).to(dev)).float().cpu().numpy()
    y_ref = O.llama_mlp(x, gu_p, gu_s, dn_p, dn_s, 128)
    scale = np.abs(y_ref).max()
    assert np.isfinite(y).all()
    assert np.abs(y - y_ref).max() <= 1e-2 * scale + 1e-2


def test_mlp_c_abi_workspace_and_errors():
    hidden, inter, M = 256, 384, 8
    x, gu_p, gu_s, dn_p, dn_s = _mlp_problem(M, hidden, inter, seed=5)
    lib = capi.load()
    dev = torch.device("cuda:0")
    t = [torch.from_numpy(a).to(dev) for a in (gu_p, gu_s, dn_p, dn_s)]
    gu = capi.Plan(0, 2 * inter, hidden, 128, 1, t[0].data_ptr(), t[1].data_ptr())
    dn = capi.Plan(0, hidden, inter, 128, 1, t[2].data_ptr(), t[3].data_ptr())
    nbytes = lib.sk_w2a8_mlp_workspace_bytes(gu.handle, dn.handle, M)
    assert nbytes > 0 and nbytes % 256 == 0
    assert lib.sk_w2a8_mlp_workspace_bytes(dn.handle, gu.handle, M) == 0          # not an MLP pair
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    d_x = torch.from_numpy(x).to(dev)
    out = torch.empty(M, hidden, dtype=torch.float16, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    assert lib.sk_w2a8_mlp_forward(gu.handle, dn.handle, M, d_x.data_ptr(), hidden, out.data_ptr(), hidden,
                                   ws.data_ptr(), nbytes - 256, st) == capi.SK_ERR_BAD_SHAPE
    assert lib.sk_w2a8_mlp_forward(gu.handle, dn.handle, M, d_x.data_ptr(), hidden, out.data_ptr(), hidden,
                                   None, nbytes, st) == capi.SK_ERR_NULL_POINTER
    assert lib.sk_w2a8_mlp_forward(gu.handle, dn.handle, M, d_x.data_ptr(), hidden, out.data_ptr(), hidden,
                                   ws.data_ptr(), nbytes, st) == 0
    torch.cuda.synchronize()
    y_ref = O.llama_mlp(x, gu_p, gu_s, dn_p, dn_s, 128)
    assert np.abs(out.float().cpu().numpy() - y_ref).max() <= 1e-2 * np.abs(y_ref).max() + 1e-2


def test_w2a8_linear_from_float_matches_dequantised_weight():
    """W2A8Linear.from_float: reference quantisation rule on the host, GEMM on the device."""
    from slimkernels_b200 import format as F
    from slimkernels_b200.torch import W2A8Linear
    rng = np.random.default_rng(3)
    w = rng.standard_normal((256, 512)).astype(np.float32) * 0.02          # [out, in]
    lin = W2A8Linear.from_float(torch.from_numpy(w), group_size=128)
    x = rng.standard_normal((5, 512)).astype(np.float16)
    y = lin(torch.from_numpy(x).cuda()).float().cpu().numpy()
    codes, scales = F.quantize_to_uint2(w.T.copy(), 128)
    wdq = F.dequantize_from_uint2(codes, scales.astype(np.float16), 128).astype(np.float32)     # [in, out]
    xq, xs = O.quantize_activation_int8(x)
    y_ref = (xq.astype(np.float32) * xs[:, None]) @ wdq
    assert np.abs(y - y_ref).max() <= 1e-2
