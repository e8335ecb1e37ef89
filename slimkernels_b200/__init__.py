"""slimkernels_b200 — B200 (sm_100a) implementation of SlimKernels' W2A8 GEMM path.

  format      host-side 2-bit packing / group quantisation (mirrors matrix_packer.py, quantization.py)
  capi        ctypes binding of the C ABI (include/sk_w2a8.h)
  torch       PyTorch op `slimkernels::w2a8_gemm`, W2A8Linear, W2A8LlamaMLP, N-sharded execution
  workloads   seeded synthetic inputs of the benchmark configurations
"""
__version__ = "0.1.0"
