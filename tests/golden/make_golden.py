"""Generates tests/golden/reference_vectors.npz from the UNMODIFIED reference modules.

Run in a container that has the reference checked out (it is not needed at test time):

    python tests/golden/make_golden.py <path of the reference checkout>

It imports matrix_packer.py and quantization.py from the reference tree, feeds them
seeded inputs and stores inputs + outputs.  The composed GEMM vectors follow the
benchmark's reference path: unpack_matrix -> dequantize_from_uint2 -> fp32 matmul,
plus exact per-group integer partials computed with int64 einsum (no oracle code).
"""
import contextlib
import io
import os
import sys

import numpy as np


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    import matrix_packer as mp        # noqa: E402  (reference module)
    import quantization as qz         # noqa: E402  (reference module)

    rng = np.random.default_rng(20240607)
    out = {}

    # ---- pack / unpack ----------------------------------------------------------
    for i, (r, c) in enumerate([(4, 8), (10, 8), (7, 64), (33, 132), (128, 256)]):
        codes = rng.integers(0, 4, size=(r, c), dtype=np.uint8)
        packed = mp.pack_matrix(codes)
        assert np.array_equal(mp.unpack_matrix(packed), codes)
        out[f"pack{i}_codes"] = codes
        out[f"pack{i}_packed"] = packed

    # ---- quantize / dequantize --------------------------------------------------
    for i, (r, c, g, dt) in enumerate([(8, 2, 8, np.float64), (16, 4, 8, np.float32),
                                       (256, 24, 128, np.float32), (64, 5, 32, np.float64),
                                       (128, 16, 128, np.float16)]):
        w = rng.standard_normal((r, c)).astype(dt)
        if i == 2:
            w[:128, 3] = 0.0                         # an all-zero group (scale floor 1e-9)
            w[5, 7] = 0.5 * np.abs(w[:128, 7]).max() / 1.5 * 1.0   # near a rounding tie
        with contextlib.redirect_stdout(io.StringIO()):          # reference prints debug arrays
            codes, scales = qz.quantize_to_uint2(w, group_size=g)
        deq = qz.dequantize_from_uint2(codes, scales, group_size=g)
        out[f"quant{i}_w"] = w
        out[f"quant{i}_g"] = np.int64(g)
        out[f"quant{i}_codes"] = codes
        out[f"quant{i}_scales"] = scales
        out[f"quant{i}_deq"] = deq

    # ---- composed W2A8 GEMM (reference format functions + fp32 matmul) ----------
    shapes = [(1, 8, 128, 128), (5, 24, 256, 128), (16, 136, 384, 128), (33, 64, 256, 64),
              (3, 40, 128, 32), (17, 130, 512, 128)]
    for i, (M, N, K, G) in enumerate(shapes):
        x_q = rng.integers(-127, 128, size=(M, K), dtype=np.int64).astype(np.int8)
        x_scale = rng.uniform(0.005, 0.02, size=(M,)).astype(np.float32)
        codes_nk = rng.integers(0, 4, size=(N, K), dtype=np.uint8)
        w_packed = mp.pack_matrix(codes_nk)
        w_scale = rng.uniform(0.001, 0.01, size=(K // G, N)).astype(np.float16)
        unp = mp.unpack_matrix(w_packed)
        wdq = qz.dequantize_from_uint2(np.ascontiguousarray(unp.T), w_scale, group_size=G)   # fp16 [K,N]
        y = (x_q.astype(np.float32) * x_scale[:, None]) @ wdq.astype(np.float32)
        part = np.einsum("mgk,ngk->gmn", x_q.astype(np.int64).reshape(M, K // G, G),
                         (unp.astype(np.int64) - 1).reshape(N, K // G, G)).astype(np.int32)
        out[f"gemm{i}_shape"] = np.array([M, N, K, G], dtype=np.int64)
        out[f"gemm{i}_x_q"] = x_q
        out[f"gemm{i}_x_scale"] = x_scale
        out[f"gemm{i}_w_packed"] = w_packed
        out[f"gemm{i}_w_scale"] = w_scale
        out[f"gemm{i}_y_ref"] = y.astype(np.float32)
        out[f"gemm{i}_partials_zp1"] = part

    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_vectors.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, os.path.getsize(dst), "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path of the reference checkout>")
    main(sys.argv[1])
