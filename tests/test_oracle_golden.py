"""Pins the CPU oracle (oracle/) to the reference: its own known-answer tests and golden vectors
generated from the unmodified reference modules (tests/golden/make_golden.py)."""
import numpy as np
import pytest

from oracle import c_oracle
from oracle import w2a8_oracle as O

# Known-answer vectors of the reference's tests, restated as literals
# (test_matrix_packer.py:7-25 / :45-61 and test_quantization.py:108-140).
KAT_CODES = np.array([[0, 1, 2, 3, 0, 1, 2, 3], [3, 2, 1, 0, 3, 2, 1, 0],
                      [1, 1, 1, 1, 2, 2, 2, 2], [0, 3, 2, 1, 3, 0, 1, 2]], dtype=np.uint8)
KAT_PACKED = np.array([[27, 27], [228, 228], [85, 170], [57, 198]], dtype=np.uint8)
KAT_QUANT_IN = np.array([[2.0, -4.0], [1.0, -2.0], [0.5, -1.0], [-2.0, 4.0], [-1.0, 2.0], [-0.5, 1.0],
                         [0.0, 0.0], [1.5, -3.0]], dtype=np.float32)
KAT_QUANT_CODES = np.array([[3, 0], [2, 0], [1, 1], [0, 3], [0, 2], [1, 1], [1, 1], [2, 0]], dtype=np.uint8)
KAT_QUANT_SCALES = np.array([[2.0 * 2 / 3, 4.0 * 2 / 3]])

IMPLS = [pytest.param(O, id="numpy"), pytest.param(c_oracle, id="c")]


@pytest.mark.parametrize("impl", IMPLS)
def test_pack_unpack_known_answers(impl):
    np.testing.assert_array_equal(impl.pack_matrix(KAT_CODES), KAT_PACKED)
    np.testing.assert_array_equal(impl.unpack_matrix(KAT_PACKED), KAT_CODES)


@pytest.mark.parametrize("impl", IMPLS)
def test_quantize_known_answer(impl):
    codes, scales = impl.quantize_to_uint2(KAT_QUANT_IN, 8)
    np.testing.assert_allclose(scales, KAT_QUANT_SCALES, rtol=1e-5)
    np.testing.assert_array_equal(codes, KAT_QUANT_CODES)


def test_oracle_error_behaviour_matches_reference():
    with pytest.raises(ValueError, match="输入矩阵的值必须在0-3之间"):
        O.pack_matrix(np.array([[0, 1, 2, 4]], dtype=np.uint8))
    with pytest.raises(ValueError, match="输入矩阵的列数必须是4的倍数"):
        O.pack_matrix(np.array([[0, 1, 2]], dtype=np.uint8))
    with pytest.raises(ValueError, match="输入矩阵必须是uint8类型"):
        O.pack_matrix(np.array([[0, 1, 2, 3]], dtype=np.float32))
    with pytest.raises(TypeError):
        O.quantize_to_uint2([[1, 2], [3, 4]])
    with pytest.raises(ValueError):
        O.quantize_to_uint2(np.zeros((10, 4)), group_size=8)
    q = np.array([[0, 1], [2, 3]], dtype=np.uint8)
    with pytest.raises(TypeError):
        O.dequantize_from_uint2(q.astype(np.float32), np.ones((1, 2)), 2)
    with pytest.raises(ValueError):
        O.dequantize_from_uint2(q, np.ones((2, 1)), 2)
    codes, scales = O.quantize_to_uint2(np.zeros((8, 2)))
    assert np.all(codes == 1) and np.all(scales > 0)


@pytest.mark.parametrize("impl", IMPLS)
def test_pack_golden(impl, golden):
    for i in range(5):
        codes, packed = golden[f"pack{i}_codes"], golden[f"pack{i}_packed"]
        np.testing.assert_array_equal(impl.pack_matrix(codes), packed)
        np.testing.assert_array_equal(impl.unpack_matrix(packed), codes)


def test_quantize_golden(golden):
    for i in range(5):
        w, g = golden[f"quant{i}_w"], int(golden[f"quant{i}_g"])
        codes, scales = O.quantize_to_uint2(w, g)
        np.testing.assert_array_equal(codes, golden[f"quant{i}_codes"])
        np.testing.assert_array_equal(scales, golden[f"quant{i}_scales"])
        assert scales.dtype == golden[f"quant{i}_scales"].dtype
        deq = O.dequantize_from_uint2(codes, scales, g)
        assert deq.dtype == np.float16
        np.testing.assert_array_equal(deq, golden[f"quant{i}_deq"])
        if w.dtype == np.float64:
            c_codes, c_scales = c_oracle.quantize_to_uint2(w, g)
            np.testing.assert_array_equal(c_codes, codes)
            np.testing.assert_array_equal(c_scales, scales)


def _gemm_cases(golden):
    i = 0
    while f"gemm{i}_shape" in golden.files:
        M, N, K, G = (int(v) for v in golden[f"gemm{i}_shape"])
        yield i, M, N, K, G
        i += 1


def test_gemm_golden_numpy(golden):
    for i, M, N, K, G in _gemm_cases(golden):
        x_q, xs = golden[f"gemm{i}_x_q"], golden[f"gemm{i}_x_scale"]
        wp, ws = golden[f"gemm{i}_w_packed"], golden[f"gemm{i}_w_scale"]
        np.testing.assert_array_equal(O.w2a8_partials(x_q, wp, G, 1), golden[f"gemm{i}_partials_zp1"])
        y_ref = golden[f"gemm{i}_y_ref"]
        np.testing.assert_allclose(O.w2a8_gemm_dequant_path(x_q, xs, wp, ws, G), y_ref, rtol=0, atol=1e-4)
        # the integer route (what the GPU computes) agrees with the reference's dequantise-then-matmul route
        assert np.abs(O.w2a8_gemm_int_path(x_q, xs, wp, ws, G) - y_ref).max() < 2e-3


def test_gemm_golden_c(golden):
    for i, M, N, K, G in _gemm_cases(golden):
        x_q, xs = golden[f"gemm{i}_x_q"], golden[f"gemm{i}_x_scale"]
        wp, ws = golden[f"gemm{i}_w_packed"], golden[f"gemm{i}_w_scale"]
        np.testing.assert_array_equal(c_oracle.w2a8_partials(x_q, wp, G, 1), golden[f"gemm{i}_partials_zp1"])
        assert np.abs(c_oracle.w2a8_gemm(x_q, xs, wp, ws, G, 1) - golden[f"gemm{i}_y_ref"]).max() < 2e-3
        codes = O.unpack_matrix(wp)
        np.testing.assert_array_equal(
            c_oracle.dequantize_from_uint2(np.ascontiguousarray(codes.T), ws, G, 1),
            O.dequantize_from_uint2(np.ascontiguousarray(codes.T), ws, G, 1))


@pytest.mark.parametrize("zp", [1, 2])
def test_numpy_and_c_oracles_agree_on_config0_slice(zp):
    """Benchmark config 0 distributions (M=16, K=4096, G=128), a 256-feature slice of N=4096."""
    rng = np.random.default_rng(0)
    M, N, K, G = 16, 256, 4096, 128
    x_q = rng.integers(-127, 128, size=(M, K), dtype=np.int8)
    xs = rng.uniform(0.005, 0.02, size=(M,)).astype(np.float32)
    wp = rng.integers(0, 256, size=(N, K // 4), dtype=np.uint8)
    ws = rng.uniform(0.001, 0.01, size=(K // G, N)).astype(np.float16)
    p_np = O.w2a8_partials(x_q, wp, G, zp)
    np.testing.assert_array_equal(p_np, c_oracle.w2a8_partials(x_q, wp, G, zp))
    assert np.abs(p_np).max() <= 128 * 127 * 2
    y_int = O.w2a8_gemm_int_path(x_q, xs, wp, ws, G, zp)
    y_deq = O.w2a8_gemm_dequant_path(x_q, xs, wp, ws, G, zp)
    assert np.abs(y_int - y_deq).max() < 2e-3
    assert np.abs(c_oracle.w2a8_gemm(x_q, xs, wp, ws, G, zp) - y_int).max() < 1e-4


def test_half_conversion_in_c_oracle_is_exact():
    rng = np.random.default_rng(3)
    codes = rng.integers(0, 4, size=(64, 33), dtype=np.uint8)
    scales = (rng.standard_normal((2, 33)) * 10.0 ** rng.integers(-7, 4, size=(2, 33))).astype(np.float16)
    np.testing.assert_array_equal(c_oracle.dequantize_from_uint2(codes, scales, 32, 1),
                                  O.dequantize_from_uint2(codes, scales, 32, 1))
