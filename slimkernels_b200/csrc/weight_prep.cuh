// GPU-side weight preparation of the W2A8 format: group-wise 2-bit quantisation followed by 4-codes-per-byte
// packing, in one pass over a float32 weight matrix W[K, N] (K = in-features, groups of G rows along K).
//
// Bit-for-bit the composition the reference performs on the host,
//     codes, scales = quantize_to_uint2(W, group_size=G)            (slimkernels/.../quantization.py:3-53)
//     w_packed      = pack_matrix(ascontiguousarray(codes.T))       (matrix_packer.py:3-36)
// for a float32 W: every step is the same IEEE single-precision operation numpy performs
//     scale = max(max_k |W[k, n]|, 1e-9f) / 1.5f                    (quantization.py:31: the 1e-9 floor)
//     code  = clip(rint(W[k, n] / scale) + 1, 0, 3)                 (round half to even; zero point 1, :43)
//     byte j of row n of w_packed = code[4j] << 6 | code[4j+1] << 4 | code[4j+2] << 2 | code[4j+3]
// (true division and rintf, so this file must not be compiled with fast-math).  The scales are written as float32
// (what quantize_to_uint2 returns) and / or as the fp16 the GEMM consumes (round to nearest even, numpy's astype).
//
// HBM-bound: reads 4 K N bytes (the second pass over a group hits L1 / L2), writes K N / 4 + 2..6 (K / G) N.
// One CTA = 128 consecutive output features x one scale group; a thread owns one feature: its reads of a row of W
// are coalesced across the CTA, its writes are 16-byte pieces of its own packed row.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sk {

constexpr int kPrepThreads = 128;

__device__ __forceinline__ uint32_t quantize_code(float x, float scale) {
  const float level = rintf(__fdiv_rn(x, scale)) + 1.0f;
  return static_cast<uint32_t>(fminf(fmaxf(level, 0.0f), 3.0f));
}

// w: float32 [K, ld_w]; w_packed: uint8 [N, K/4]; scale_f32 / scale_f16: [K/G, N] (either may be null).
// G % 4 == 0, K % G == 0.  grid = (ceil(N / 128), K / G).
__global__ void __launch_bounds__(kPrepThreads)
quantize_pack_weight_kernel(const float* __restrict__ w, long long ld_w, int K, int N, int G,
                            uint8_t* __restrict__ w_packed, float* __restrict__ scale_f32,
                            __half* __restrict__ scale_f16) {
  const int n = blockIdx.x * kPrepThreads + threadIdx.x;
  const int g = blockIdx.y;
  if (n >= N) return;
  const float* col = w + static_cast<long long>(g) * G * ld_w + n;
  float amax = 0.0f;
  for (int k = 0; k < G; ++k) amax = fmaxf(amax, fabsf(col[static_cast<long long>(k) * ld_w]));
  const float scale = __fdiv_rn(fmaxf(amax, 1e-9f), 1.5f);
  if (scale_f32) scale_f32[static_cast<long long>(g) * N + n] = scale;
  if (scale_f16) scale_f16[static_cast<long long>(g) * N + n] = __float2half_rn(scale);

  uint8_t* dst = w_packed + static_cast<long long>(n) * (K / 4) + static_cast<long long>(g) * (G / 4);
  const bool vec = (G % 64) == 0 && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
  if (vec) {
    for (int k0 = 0; k0 < G; k0 += 64) {          // 64 codes -> 16 bytes
      uint32_t words[4];
#pragma unroll
      for (int wd = 0; wd < 4; ++wd) {
        uint32_t word = 0;
#pragma unroll
        for (int b = 0; b < 4; ++b) {             // byte b of the word: codes k0 + 16 wd + 4 b .. + 3
          uint32_t byte = 0;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            byte = (byte << 2) | quantize_code(col[static_cast<long long>(k0 + 16 * wd + 4 * b + j) * ld_w], scale);
          word |= byte << (8 * b);
        }
        words[wd] = word;
      }
      *reinterpret_cast<uint4*>(dst + k0 / 4) = make_uint4(words[0], words[1], words[2], words[3]);
    }
  } else {
    for (int k0 = 0; k0 < G; k0 += 4) {
      uint32_t byte = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) byte = (byte << 2) | quantize_code(col[static_cast<long long>(k0 + j) * ld_w], scale);
      dst[k0 / 4] = static_cast<uint8_t>(byte);
    }
  }
}

}  // namespace sk
