"""Host-side weight format of the W2A8 path: 2-bit packing and group-wise quantisation.

Drop-in mirrors of the reference's numpy helpers, same names, argument meaning and error
behaviour, vectorised (the reference loops over byte columns in Python):

* ``pack_matrix`` / ``unpack_matrix``      <- matrix_packer.py:3-36 / :38-66
* ``quantize_to_uint2``                     <- quantization.py:3-53  (without its debug prints, :44-45)
* ``dequantize_from_uint2``                 <- quantization.py:55-93

plus ``prepare_weight`` which composes them into the operand layout the GEMM consumes:
``w_packed`` uint8 [N, K/4] (K packed, 4 codes per byte, first code in bits 7:6) and
``w_scale`` fp16 [K/G, N].
"""
from __future__ import annotations

import numpy as np

ZERO_POINT = 1          # quantization.py:43 and :89 — stored code c means c - 1
_QUANT_MAX = 3          # 2 bits


def pack_matrix(input_matrix: np.ndarray) -> np.ndarray:
    """Pack every 4 columns of a uint8 matrix of 2-bit codes into one byte (matrix_packer.py:3)."""
    if input_matrix.dtype != np.uint8:
        raise ValueError("输入矩阵必须是uint8类型")
    if input_matrix.shape[1] % 4 != 0:
        raise ValueError("输入矩阵的列数必须是4的倍数")
    if input_matrix.size and int(input_matrix.max()) > _QUANT_MAX:
        raise ValueError("输入矩阵的值必须在0-3之间")
    rows, cols = input_matrix.shape
    quads = input_matrix.reshape(rows, cols // 4, 4)
    out = quads[:, :, 3].copy()
    for i, shift in enumerate((6, 4, 2)):                     # first column of a quad in the top bits
        out |= quads[:, :, i] << shift
    return out


def unpack_matrix(packed_matrix: np.ndarray) -> np.ndarray:
    """Inverse of ``pack_matrix``: one byte -> 4 columns of codes 0..3 (matrix_packer.py:38)."""
    if packed_matrix.dtype != np.uint8:
        raise ValueError("输入矩阵必须是uint8类型")
    shifts = np.array([6, 4, 2, 0], dtype=np.uint8)
    codes = (packed_matrix[:, :, None] >> shifts) & np.uint8(3)
    return np.ascontiguousarray(codes.reshape(packed_matrix.shape[0], -1))


def quantize_to_uint2(matrix: np.ndarray, group_size: int = 8):
    """Group-wise (groups of ``group_size`` rows) quantisation to codes 0..3 (quantization.py:3).

    scale = max(max|x|, 1e-9) / 1.5 per (group, column); code = clip(round(x/scale) + 1, 0, 3)
    with numpy's round-half-to-even.  Returns (codes uint8 [R, C], scales [R/g, C]).
    """
    if not isinstance(matrix, np.ndarray):
        raise TypeError("Input must be a numpy array")
    num_rows, num_cols = matrix.shape
    if num_rows % group_size != 0:
        raise ValueError(
            f"Number of rows ({num_rows}) must be divisible by group_size ({group_size})")
    grouped = matrix.reshape(num_rows // group_size, group_size, num_cols)
    scales = np.maximum(np.abs(grouped).max(axis=1), 1e-9) / (_QUANT_MAX / 2)
    levels = np.round(grouped / scales[:, None, :]) + ZERO_POINT
    codes = np.clip(levels, 0, _QUANT_MAX).astype(np.uint8).reshape(num_rows, num_cols)
    return codes, scales


def dequantize_from_uint2(quantized: np.ndarray, scales: np.ndarray, group_size: int = 8) -> np.ndarray:
    """(code - 1) * scale per group, returned as float16 (quantization.py:55)."""
    if not isinstance(quantized, np.ndarray) or not isinstance(scales, np.ndarray):
        raise TypeError("Both inputs must be numpy arrays")
    if quantized.dtype != np.uint8:
        raise TypeError("Quantized matrix must be of type uint8")
    num_rows, num_cols = quantized.shape
    if num_rows % group_size != 0:
        raise ValueError(
            f"Number of rows ({num_rows}) must be divisible by group_size ({group_size})")
    expected = (num_rows // group_size, num_cols)
    if scales.shape != expected:
        raise ValueError(f"Scales shape {scales.shape} does not match expected shape {expected}")
    values = quantized.reshape(expected[0], group_size, num_cols).astype(np.float32) - ZERO_POINT
    return (values * scales[:, None, :]).reshape(num_rows, num_cols).astype(np.float16)


def prepare_weight(weight_kn: np.ndarray, group_size: int = 128):
    """float W[K, N] -> (w_packed uint8 [N, K/4], w_scale float16 [K/G, N]).

    Groups run along K (the row axis handed to ``quantize_to_uint2``); packing runs along K of
    the transposed code matrix, so byte j of row n holds k = 4j..4j+3 with k = 4j in bits 7:6.
    This is the K-packed orientation of the reference's prototype kernel (a_k = b_k / 4,
    wgmma_sm90_W2A8.cu:530-531).
    """
    codes_kn, scales = quantize_to_uint2(np.asarray(weight_kn), group_size)
    w_packed = pack_matrix(np.ascontiguousarray(codes_kn.T))
    return w_packed, scales.astype(np.float16)


# --------------------------------------------------------------------------------------------------
# Serialised container of one quantised weight (the on-disk form of the operand pair).  The reference has
# none (its helpers only return arrays); this one is little-endian and self-describing:
#   bytes 0..7    magic  b"SKW2A8" + b"\x00" + version byte (1)
#   5 x int64     N (out-features), K (in-features), group_size, zero_point, scale dtype code (2 = float16)
#   N * K / 4     w_packed, matrix_packer layout (row n, byte j = codes k = 4j .. 4j+3, k = 4j in bits 7:6)
#   K/G * N * 2   w_scale, float16 [K/G, N]
#   uint32        CRC-32 of every byte before it
# --------------------------------------------------------------------------------------------------
_MAGIC = b"SKW2A8\x00\x01"


def dumps_weight(w_packed: np.ndarray, w_scale: np.ndarray, group_size: int, zero_point: int = ZERO_POINT) -> bytes:
    """Serialise (w_packed uint8 [N, K/4], w_scale float16 [K/G, N]) into the container described above."""
    import struct
    import zlib
    if w_packed.dtype != np.uint8 or w_packed.ndim != 2:
        raise TypeError("w_packed must be a 2-D uint8 array")
    if w_scale.dtype != np.float16 or w_scale.ndim != 2:
        raise TypeError("w_scale must be a 2-D float16 array")
    N, K = w_packed.shape[0], w_packed.shape[1] * 4
    if group_size <= 0 or K % group_size or w_scale.shape != (K // group_size, N):
        raise ValueError(f"w_scale shape {w_scale.shape} does not match ({K // max(group_size, 1)}, {N})")
    if not 0 <= zero_point <= 3:
        raise ValueError("zero_point must be in 0..3")
    body = (_MAGIC + struct.pack("<5q", N, K, group_size, zero_point, 2) +
            np.ascontiguousarray(w_packed).tobytes() + np.ascontiguousarray(w_scale).astype("<f2").tobytes())
    return body + struct.pack("<I", zlib.crc32(body) & 0xFFFFFFFF)


def loads_weight(blob: bytes) -> dict:
    """Inverse of ``dumps_weight``: {"w_packed", "w_scale", "group_size", "zero_point"}; ValueError if damaged."""
    import struct
    import zlib
    head = len(_MAGIC) + 40
    if len(blob) < head + 4 or blob[:len(_MAGIC) - 1] != _MAGIC[:-1]:
        raise ValueError("not a W2A8 weight container")
    if blob[len(_MAGIC) - 1] != _MAGIC[-1]:
        raise ValueError(f"unsupported container version {blob[len(_MAGIC) - 1]}")
    N, K, G, zp, sdt = struct.unpack("<5q", blob[len(_MAGIC):head])
    if N <= 0 or K <= 0 or G <= 0 or K % 4 or K % G or not 0 <= zp <= 3 or sdt != 2:
        raise ValueError("inconsistent container header")
    n_packed, n_scale = N * K // 4, (K // G) * N * 2
    if len(blob) != head + n_packed + n_scale + 4:
        raise ValueError("container length does not match its header")
    (crc,) = struct.unpack("<I", blob[-4:])
    if crc != (zlib.crc32(blob[:-4]) & 0xFFFFFFFF):
        raise ValueError("container checksum mismatch")
    w_packed = np.frombuffer(blob, dtype=np.uint8, count=n_packed, offset=head).reshape(N, K // 4).copy()
    w_scale = np.frombuffer(blob, dtype="<f2", count=n_scale // 2, offset=head + n_packed).reshape(K // G, N)
    return {"w_packed": w_packed, "w_scale": w_scale.astype(np.float16), "group_size": int(G), "zero_point": int(zp)}


def save_weight(path, w_packed, w_scale, group_size, zero_point=ZERO_POINT) -> None:
    with open(path, "wb") as f:
        f.write(dumps_weight(w_packed, w_scale, group_size, zero_point))


def load_weight(path) -> dict:
    with open(path, "rb") as f:
        return loads_weight(f.read())


# --------------------------------------------------------------------------------------------------
# Tiled weight order consumed by the sm_100a kernel (a pure permutation of the 2-bit codes).
# Block (tile T of 128 rows, k-block B of 128 codes) is 4096 bytes at (T * k_blocks + B) * 4096; the
# little-endian 32-bit word of (row r, 16-code chunk c) sits at byte (c // 4) * 2048 + r * 16 + (c % 4) * 4
# and holds  sum_{j,b} code[128 T + r, 128 B + 16 c + 4 j + b] << (4 b + 2 (j & 1) + 16 (j >> 1)).
# N is padded to a multiple of 128 and K to a multiple of 128 with code 0.
# --------------------------------------------------------------------------------------------------
_j, _b = np.arange(4)[:, None], np.arange(4)[None, :]
_TILED_SHIFTS = (4 * _b + 2 * (_j & 1) + 16 * (_j >> 1)).astype(np.uint32)   # [j, b]


def tiled_nbytes(N: int, K: int) -> int:
    return ((N + 127) // 128) * ((K + 127) // 128) * 4096


def repack_tiled(w_packed: np.ndarray) -> np.ndarray:
    """uint8 [N, K/4] in ``pack_matrix`` layout -> uint8 [tiled_nbytes] in the kernel's tile order."""
    N, K = w_packed.shape[0], w_packed.shape[1] * 4
    T, B = (N + 127) // 128, (K + 127) // 128
    codes = np.zeros((T * 128, B * 128), dtype=np.uint32)
    codes[:N, :K] = unpack_matrix(w_packed)
    c6 = codes.reshape(T, 128, B, 8, 4, 4)                       # [T, r, B, c, j, b]
    shifts = _TILED_SHIFTS
    words = (c6 << shifts).sum(axis=(4, 5), dtype=np.uint32)     # [T, r, B, c]
    words = words.reshape(T, 128, B, 2, 4).transpose(0, 2, 3, 1, 4)   # [T, B, half, r, c % 4]
    return np.ascontiguousarray(words).astype("<u4").view(np.uint8).reshape(-1)


def unrepack_tiled(w_tiled: np.ndarray, N: int, K: int) -> np.ndarray:
    """Inverse of ``repack_tiled``: back to uint8 [N, K/4] in ``pack_matrix`` layout."""
    T, B = (N + 127) // 128, (K + 127) // 128
    words = np.ascontiguousarray(w_tiled).view("<u4").reshape(T, B, 2, 128, 4).astype(np.uint32)
    words = words.transpose(0, 3, 1, 2, 4).reshape(T, 128, B, 8)  # [T, r, B, c]
    shifts = _TILED_SHIFTS
    codes = ((words[..., None, None] >> shifts) & 3).astype(np.uint8)   # [T, r, B, c, j, b]
    codes = codes.reshape(T * 128, B * 128)[:N, :K]
    return pack_matrix(np.ascontiguousarray(codes))
