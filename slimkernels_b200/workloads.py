"""Seeded synthetic inputs with the shapes and value distributions of the W2A8 benchmark configs.

Draw order (fixed): x_q, x_scale, codes, w_scale — from numpy's PCG64 seeded with ``seed``:
  x_q     int8  [M, K]     uniform integers in [-127, 127]
  x_scale fp32  [M]        uniform [0.005, 0.02]
  codes   uint8 [N, K]     uniform integers 0..3, packed 4 per byte along K (first code in bits 7:6)
  w_scale fp16  [K/G, N]   uniform [0.001, 0.01]
"""
from __future__ import annotations

import numpy as np

from .format import pack_matrix

# Llama-2-7B linear layers as (N, K): fused QKV, O-proj, fused gate+up, down.
LLAMA2_7B_SHAPES = {"qkv": (12288, 4096), "o_proj": (4096, 4096), "gate_up": (22016, 4096),
                    "down": (4096, 11008)}
DECODE_M = (1, 4, 8, 16, 32)
PREFILL_M = (2048, 4096, 8192)
PREFILL_NK = (8192, 8192)
# Llama-3-70B MLP layers as (N, K): fused gate+up, down.
LLAMA3_70B_MLP = {"gate_up": (57344, 8192), "down": (8192, 28672)}


def make_weight(N: int, K: int, group_size: int = 128, seed: int = 0, rng=None):
    """(w_packed uint8 [N, K/4], w_scale fp16 [K/G, N]) with the benchmark's distributions."""
    rng = rng if rng is not None else np.random.default_rng(seed)
    w_packed = np.empty((N, K // 4), dtype=np.uint8)
    step = max(1, (1 << 24) // K)
    for r0 in range(0, N, step):                      # bounded temporary: codes are 4x the packed size
        codes = rng.integers(0, 4, size=(min(step, N - r0), K), dtype=np.uint8)
        w_packed[r0:r0 + codes.shape[0]] = pack_matrix(codes)
    w_scale = rng.uniform(0.001, 0.01, size=(K // group_size, N)).astype(np.float16)
    return w_packed, w_scale


def make_activation(M: int, K: int, seed: int = 0, rng=None):
    """(x_q int8 [M, K], x_scale fp32 [M]) with the benchmark's distributions."""
    rng = rng if rng is not None else np.random.default_rng(seed)
    x_q = rng.integers(-127, 128, size=(M, K), dtype=np.int8)
    x_scale = rng.uniform(0.005, 0.02, size=(M,)).astype(np.float32)
    return x_q, x_scale


def make_problem(M: int, N: int, K: int, group_size: int = 128, seed: int = 0):
    """All four operands of one GEMM, drawn in the documented order from one generator."""
    rng = np.random.default_rng(seed)
    x_q, x_scale = make_activation(M, K, rng=rng)
    w_packed, w_scale = make_weight(N, K, group_size, rng=rng)
    return x_q, x_scale, w_packed, w_scale
