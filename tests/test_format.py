"""Host-side format module (slimkernels_b200/format.py) against the reference's known answers, the golden
vectors and the oracle; same cases as the reference's test_matrix_packer.py / test_quantization.py."""
import numpy as np
import pytest

from oracle import w2a8_oracle as O
from slimkernels_b200 import format as F
from slimkernels_b200 import workloads as W

from test_oracle_golden import (KAT_CODES, KAT_PACKED, KAT_QUANT_CODES, KAT_QUANT_IN, KAT_QUANT_SCALES)


def test_pack_unpack_known_answers():
    np.testing.assert_array_equal(F.pack_matrix(KAT_CODES), KAT_PACKED)
    np.testing.assert_array_equal(F.unpack_matrix(KAT_PACKED), KAT_CODES)


def test_pack_invalid_input():
    with pytest.raises(ValueError, match="输入矩阵的值必须在0-3之间"):
        F.pack_matrix(np.array([[0, 1, 2, 4]], dtype=np.uint8))
    with pytest.raises(ValueError, match="输入矩阵的列数必须是4的倍数"):
        F.pack_matrix(np.array([[0, 1, 2]], dtype=np.uint8))
    with pytest.raises(ValueError, match="输入矩阵必须是uint8类型"):
        F.pack_matrix(np.array([[0, 1, 2, 3]], dtype=np.float32))
    with pytest.raises(ValueError, match="输入矩阵必须是uint8类型"):
        F.unpack_matrix(np.array([[0, 1]], dtype=np.int32))


def test_pack_unpack_roundtrip_and_golden(golden):
    rng = np.random.default_rng(7)
    original = rng.integers(0, 4, (10, 8), dtype=np.uint8)
    np.testing.assert_array_equal(F.unpack_matrix(F.pack_matrix(original)), original)
    for i in range(5):
        np.testing.assert_array_equal(F.pack_matrix(golden[f"pack{i}_codes"]), golden[f"pack{i}_packed"])
        np.testing.assert_array_equal(F.unpack_matrix(golden[f"pack{i}_packed"]), golden[f"pack{i}_codes"])
    empty = np.zeros((0, 8), dtype=np.uint8)
    assert F.pack_matrix(empty).shape == (0, 2)


def test_quantize_basic_shapes_and_errors():
    m = np.arange(16, dtype=np.float64).reshape(8, 2) - 7.5
    q, s = F.quantize_to_uint2(m, group_size=8)
    assert q.dtype == np.uint8 and q.min() >= 0 and q.max() <= 3 and s.shape == (1, 2)
    with pytest.raises(TypeError):
        F.quantize_to_uint2([[1, 2], [3, 4]])
    with pytest.raises(ValueError):
        F.quantize_to_uint2(np.random.randn(10, 4), group_size=8)
    q, s = F.quantize_to_uint2(np.zeros((8, 2)))
    assert np.all(q == 1) and np.all(s > 0)
    q, s = F.quantize_to_uint2(np.random.randn(16, 4), group_size=8)
    assert s.shape == (2, 4) and q.shape == (16, 4)


def test_quantize_known_answer_and_golden(golden):
    q, s = F.quantize_to_uint2(KAT_QUANT_IN, group_size=8)
    np.testing.assert_allclose(s, KAT_QUANT_SCALES, rtol=1e-5)
    np.testing.assert_array_equal(q, KAT_QUANT_CODES)
    for i in range(5):
        w, g = golden[f"quant{i}_w"], int(golden[f"quant{i}_g"])
        q, s = F.quantize_to_uint2(w, g)
        np.testing.assert_array_equal(q, golden[f"quant{i}_codes"])
        np.testing.assert_array_equal(s, golden[f"quant{i}_scales"])
        np.testing.assert_array_equal(F.dequantize_from_uint2(q, s, g), golden[f"quant{i}_deq"])


def test_dequantize_invalid_input():
    q = np.array([[0, 1], [2, 3]], dtype=np.uint8)
    s = np.array([[1.0, 1.0]])
    with pytest.raises(TypeError):
        F.dequantize_from_uint2([[0, 1], [2, 3]], s)
    with pytest.raises(TypeError):
        F.dequantize_from_uint2(q, [[1.0, 1.0]])
    with pytest.raises(TypeError):
        F.dequantize_from_uint2(q.astype(np.float32), s)
    with pytest.raises(ValueError):
        F.dequantize_from_uint2(q, np.array([[1.0], [1.0]]), group_size=2)
    out = F.dequantize_from_uint2(q, s, group_size=2)
    assert out.dtype == np.float16 and out.shape == (2, 2)


def test_prepare_weight_composition():
    rng = np.random.default_rng(11)
    K, N, G = 256, 24, 128
    w = rng.standard_normal((K, N)).astype(np.float32)
    w_packed, w_scale = F.prepare_weight(w, G)
    assert w_packed.shape == (N, K // 4) and w_packed.dtype == np.uint8
    assert w_scale.shape == (K // G, N) and w_scale.dtype == np.float16
    codes_kn, scales = O.quantize_to_uint2(w, G)
    np.testing.assert_array_equal(O.unpack_matrix(w_packed), codes_kn.T)
    np.testing.assert_array_equal(w_scale, scales.astype(np.float16))
    # byte layout: code k = 4j in bits 7:6
    n, j = 5, 9
    b = int(w_packed[n, j])
    assert [(b >> s) & 3 for s in (6, 4, 2, 0)] == [int(codes_kn[4 * j + i, n]) for i in range(4)]


@pytest.mark.parametrize("N,K", [(128, 128), (200, 160), (5, 32), (384, 512), (130, 96), (1, 4096)])
def test_tiled_repack_round_trip_against_matrix_packer(N, K):
    """repack is a pure permutation: unpack(unrepack(repack(p))) == unpack(p), with the oracle's unpack."""
    rng = np.random.default_rng(N * 1000 + K)
    codes = rng.integers(0, 4, size=(N, K), dtype=np.uint8)
    p = O.pack_matrix(codes)
    t = F.repack_tiled(p)
    assert t.dtype == np.uint8 and t.size == F.tiled_nbytes(N, K)
    back = F.unrepack_tiled(t, N, K)
    np.testing.assert_array_equal(O.unpack_matrix(back), codes)
    # word semantics the kernel relies on: every nibble of a word holds two codes (byte-permute selectors)
    words = t.view("<u4")
    kb = (K + 127) // 128
    for (n, k0) in [(0, 0), (N - 1, ((K - 16) // 16) * 16), (N // 2, (K // 32) * 16)]:
        T, r, B, c = n // 128, n % 128, k0 // 128, (k0 % 128) // 16
        w = int(words[(T * kb + B) * 1024 + (c // 4) * 512 + r * 4 + (c % 4)])
        got = [(w >> (4 * b + 2 * (j & 1) + 16 * (j >> 1))) & 3 for j in range(4) for b in range(4)]
        assert got == [int(v) for v in codes[n, k0:k0 + 16]]


def test_workload_generator_is_seeded_and_in_range():
    a = W.make_problem(5, 130, 256, 128, seed=0)
    b = W.make_problem(5, 130, 256, 128, seed=0)
    for u, v in zip(a, b):
        np.testing.assert_array_equal(u, v)
    x_q, x_scale, w_packed, w_scale = a
    assert x_q.dtype == np.int8 and x_q.min() >= -127 and x_q.max() <= 127
    assert x_scale.dtype == np.float32 and 0.005 <= x_scale.min() and x_scale.max() <= 0.02
    assert w_packed.shape == (130, 64) and w_scale.shape == (2, 130) and w_scale.dtype == np.float16
    assert 0.001 <= float(w_scale.min()) and float(w_scale.max()) <= 0.01


def test_weight_container_round_trip_and_damage(tmp_path):
    rng = np.random.default_rng(11)
    w = rng.standard_normal((256, 40)).astype(np.float32)           # K = 256, N = 40
    w_packed, w_scale = F.prepare_weight(w, 64)
    blob = F.dumps_weight(w_packed, w_scale, 64)
    back = F.loads_weight(blob)
    np.testing.assert_array_equal(back["w_packed"], w_packed)
    np.testing.assert_array_equal(back["w_scale"].view(np.uint16), w_scale.view(np.uint16))
    assert back["group_size"] == 64 and back["zero_point"] == 1
    F.save_weight(tmp_path / "w.skw", w_packed, w_scale, 64, zero_point=2)
    assert F.load_weight(tmp_path / "w.skw")["zero_point"] == 2
    damaged = bytearray(blob)
    damaged[60] ^= 0x10
    with pytest.raises(ValueError, match="checksum"):
        F.loads_weight(bytes(damaged))
    with pytest.raises(ValueError, match="length"):
        F.loads_weight(blob[:-5] + blob[-4:])
    with pytest.raises(ValueError, match="not a W2A8"):
        F.loads_weight(b"x" * 100)
    with pytest.raises(ValueError):
        F.dumps_weight(w_packed, w_scale, 128)                      # scales do not match the group size
    with pytest.raises(TypeError):
        F.dumps_weight(w_packed.astype(np.int8), w_scale, 64)
