"""CPU oracle for the W2A8 GEMM path (TEST INFRASTRUCTURE, not product code).

This module restates, in plain numpy, the numerically defining pieces of the
reference (wanghaoshuang/SlimKernels) for the 2-bit-weight x int8-activation
GEMM, plus the contraction that composes them.  It exists only so that tests,
the smoke check and the CPU-baseline leg of the benchmark can check and time
the product against it; the product package never imports it.

Parity status: the *format layer* (byte layout, zero-point, scale rule,
rounding, fp16 dequantisation) is pinned by the reference's own known-answer
tests (test_matrix_packer.py:5-61, test_quantization.py:108-140) and by golden
vectors generated from the unmodified reference modules (tests/golden/).  The
reference holds no test, fixture or recorded output of a W2A8 *GEMM result*
(its CUDA prototype discards its output, wgmma_sm90_W2A8.cu:404-408), so at
the GEMM level parity is "unpinned" by the reference itself: it is anchored on
composing the reference's own format functions with a dense fp32 matmul.

Every function cites the reference lines it follows.
"""
from __future__ import annotations

import numpy as np

# Reference constant: stored code c means (c - 1)   (quantization.py:43, :89)
REFERENCE_ZERO_POINT = 1


# --------------------------------------------------------------------------- #
# matrix_packer.py
# --------------------------------------------------------------------------- #
def pack_matrix(input_matrix: np.ndarray) -> np.ndarray:
    """u8 codes [R, C] -> u8 bytes [R, C/4]; first column in the top bits.

    Follows matrix_packer.py:3-36: dtype / column-count / range checks in that
    order (:13-21) and ``c0<<6 | c1<<4 | c2<<2 | c3`` (:33-34).
    """
    if input_matrix.dtype != np.uint8:
        raise ValueError("输入矩阵必须是uint8类型")
    if input_matrix.shape[1] % 4 != 0:
        raise ValueError("输入矩阵的列数必须是4的倍数")
    if np.any(input_matrix > 3):
        raise ValueError("输入矩阵的值必须在0-3之间")
    q = input_matrix.reshape(input_matrix.shape[0], -1, 4)
    return ((q[:, :, 0] << 6) | (q[:, :, 1] << 4) | (q[:, :, 2] << 2) | q[:, :, 3]).astype(np.uint8)


def unpack_matrix(packed_matrix: np.ndarray) -> np.ndarray:
    """u8 bytes [R, C] -> u8 codes [R, 4C]   (matrix_packer.py:38-66; shifts 6,4,2,0 at :61-64)."""
    if packed_matrix.dtype != np.uint8:
        raise ValueError("输入矩阵必须是uint8类型")
    out = np.empty((packed_matrix.shape[0], packed_matrix.shape[1], 4), dtype=np.uint8)
    out[:, :, 0] = (packed_matrix >> 6) & 3
    out[:, :, 1] = (packed_matrix >> 4) & 3
    out[:, :, 2] = (packed_matrix >> 2) & 3
    out[:, :, 3] = packed_matrix & 3
    return out.reshape(packed_matrix.shape[0], -1)


# --------------------------------------------------------------------------- #
# quantization.py
# --------------------------------------------------------------------------- #
def quantize_to_uint2(matrix: np.ndarray, group_size: int = 8):
    """float [R, C] -> (u8 codes [R, C], scales [R/g, C]); groups run along rows.

    Follows quantization.py:3-53: scale = max(absmax, 1e-9) / 1.5 (:29-38),
    code = clip(round_half_even(x / scale) + 1, 0, 3) (:43-46).  The reference
    prints two debug arrays (:44-45); the oracle does not.
    """
    if not isinstance(matrix, np.ndarray):
        raise TypeError("Input must be a numpy array")
    num_rows, num_cols = matrix.shape
    if num_rows % group_size != 0:
        raise ValueError(
            f"Number of rows ({num_rows}) must be divisible by group_size ({group_size})")
    num_groups = num_rows // group_size
    reshaped = matrix.reshape(num_groups, group_size, num_cols)
    scales = np.max(np.abs(reshaped), axis=1)
    scales = np.maximum(scales, 1e-9)
    quant_range = 2 ** 2 - 1
    scales = scales / (quant_range / 2)
    q = np.clip(np.round(reshaped / scales[:, np.newaxis, :]) + REFERENCE_ZERO_POINT, 0, quant_range)
    return q.astype(np.uint8).reshape(-1, num_cols)[:num_rows], scales


def dequantize_from_uint2(quantized: np.ndarray, scales: np.ndarray, group_size: int = 8,
                          zero_point: int = REFERENCE_ZERO_POINT) -> np.ndarray:
    """(u8 codes [R, C], scales [R/g, C]) -> fp16 [R, C] = (code - zp) * scale.

    Follows quantization.py:55-93 (checks :64-80, arithmetic in fp32 :89-90,
    cast to fp16 :93).  ``zero_point`` is 1 in the reference; the argument is
    the one extension (the benchmark spec words the codes as {-2..1} = zp 2).
    """
    if not isinstance(quantized, np.ndarray) or not isinstance(scales, np.ndarray):
        raise TypeError("Both inputs must be numpy arrays")
    if quantized.dtype != np.uint8:
        raise TypeError("Quantized matrix must be of type uint8")
    num_rows, num_cols = quantized.shape
    if num_rows % group_size != 0:
        raise ValueError(
            f"Number of rows ({num_rows}) must be divisible by group_size ({group_size})")
    num_groups = num_rows // group_size
    if scales.shape != (num_groups, num_cols):
        raise ValueError(
            f"Scales shape {scales.shape} does not match expected shape {(num_groups, num_cols)}")
    rq = quantized.reshape(num_groups, group_size, num_cols)
    deq = (rq.astype(np.float32) - zero_point) * scales[:, np.newaxis, :]
    return deq.reshape(num_rows, num_cols).astype(np.float16)


# --------------------------------------------------------------------------- #
# Composition (reference holds no GEMM; this is the composed path of the
# benchmark's config 0: quantization.py + matrix_packer.py + dense matmul)
# --------------------------------------------------------------------------- #
def w2a8_partials(x_q: np.ndarray, w_packed: np.ndarray, group_size: int = 128,
                  zero_point: int = REFERENCE_ZERO_POINT) -> np.ndarray:
    """Per-group integer partial sums P[g, m, n] (int32), exact.

    P[g,m,n] = sum_{k in group g} int32(x_q[m,k]) * (int32(code[n,k]) - zp),
    code = unpack_matrix(w_packed) (matrix_packer.py:38-66), value = code - zp
    (quantization.py:89-90).  Each group sum is bounded by 128*127*2 < 2**24,
    so the float32 matmul used here per group is exact integer arithmetic.
    """
    M, K = x_q.shape
    N = w_packed.shape[0]
    assert w_packed.shape[1] * 4 == K and K % group_size == 0
    codes = unpack_matrix(w_packed).astype(np.float32) - np.float32(zero_point)   # [N, K]
    xf = x_q.astype(np.float32)
    G = group_size
    out = np.empty((K // G, M, N), dtype=np.int32)
    exact_f32 = G * 127 * max(abs(3 - zero_point), abs(zero_point)) < 2 ** 24
    for g in range(K // G):
        a = xf[:, g * G:(g + 1) * G]
        b = codes[:, g * G:(g + 1) * G]
        if exact_f32:
            out[g] = (a @ b.T).astype(np.int32)
        else:
            out[g] = (a.astype(np.float64) @ b.T.astype(np.float64)).astype(np.int32)
    return out


def w2a8_gemm_int_path(x_q, x_scale, w_packed, w_scale, group_size=128,
                       zero_point=REFERENCE_ZERO_POINT) -> np.ndarray:
    """fp32 [M, N]: x_scale[m] * sum_g w_scale[g,n] * fp32(P[g,m,n]), g ascending.

    The arithmetic the GPU kernel performs: integer group partials, scaled and
    accumulated in fp32 in group order, activation scale applied last.
    """
    P = w2a8_partials(x_q, w_packed, group_size, zero_point)
    acc = np.zeros(P.shape[1:], dtype=np.float32)
    ws = w_scale.astype(np.float32)
    for g in range(P.shape[0]):
        acc += ws[g][None, :] * P[g].astype(np.float32)
    return acc * x_scale.astype(np.float32)[:, None]


def w2a8_gemm_dequant_path(x_q, x_scale, w_packed, w_scale, group_size=128,
                           zero_point=REFERENCE_ZERO_POINT) -> np.ndarray:
    """fp32 [M, N] by the reference's own route: unpack -> dequantise -> fp32 matmul.

    codes = unpack_matrix(w_packed)                (matrix_packer.py:38)
    Wdq   = dequantize_from_uint2(codes.T, ...)    (quantization.py:55; fp16, exact for fp16 scales)
    Y     = (x_q * x_scale[:, None]) @ Wdq         (dense fp32 matmul, BLAS)
    This is the tolerance anchor: |GPU - Y| <= 1e-2 max-abs.
    """
    codes = unpack_matrix(w_packed)
    wdq = dequantize_from_uint2(np.ascontiguousarray(codes.T), w_scale, group_size, zero_point)
    xs = x_q.astype(np.float32) * x_scale.astype(np.float32)[:, None]
    return xs @ wdq.astype(np.float32)


# --------------------------------------------------------------------------- #
# Activation quantiser / MLP block.  The reference has NO activation
# quantiser; these definitions are this project's and are stated here so the
# GPU kernels have a CPU statement to be compared with.
# --------------------------------------------------------------------------- #
def quantize_activation_int8(x: np.ndarray):
    """Per-token symmetric int8: s = max|x|/127 (1.0 if the row is all zero... see code),
    q = clip(round_half_even(x / s), -127, 127).  x fp16/fp32 [M, K] -> (int8 [M,K], fp32 [M])."""
    xf = x.astype(np.float32)
    amax = np.max(np.abs(xf), axis=1)
    s = np.where(amax > 0, amax / np.float32(127.0), np.float32(1.0)).astype(np.float32)
    q = np.clip(np.rint(xf / s[:, None]), -127, 127).astype(np.int8)
    return q, s


def llama_mlp(x, gate_up_packed, gate_up_scale, down_packed, down_scale, group_size=128,
              zero_point=REFERENCE_ZERO_POINT):
    """fp32 [M, hidden] of the W2A8 Llama MLP block.

    x fp16 [M, hidden] -> int8 quant -> fused gate+up GEMM ([2*inter, hidden] packed,
    gate rows first) -> fp16 -> SiLU(gate)*up in fp32 -> int8 quant -> down GEMM.
    Intermediate GEMM outputs are rounded to fp16 as the GPU op does.
    """
    xq, xs = quantize_activation_int8(x)
    gu = w2a8_gemm_int_path(xq, xs, gate_up_packed, gate_up_scale, group_size, zero_point)
    gu = gu.astype(np.float16).astype(np.float32)
    inter = gu.shape[1] // 2
    g, u = gu[:, :inter], gu[:, inter:]
    h = (g / (1.0 + np.exp(-g))) * u
    hq, hs = quantize_activation_int8(h.astype(np.float32))
    return w2a8_gemm_int_path(hq, hs, down_packed, down_scale, group_size, zero_point)
