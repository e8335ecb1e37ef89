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
// HBM-bound: reads 4 K N bytes once, writes K N / 4 + 2..6 (K / G) N.
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

// The same code without the division, the rounding instruction or the float -> int conversion (~10 instructions for
// the division; rint and cvt issue at an eighth of the FMA rate; one of each per weight otherwise):
//   * t = x * (1 / scale) differs from the rounded quotient by a few units in the last place (< 1e-6 at |t| <= 1.5),
//     so rint(t) equals rint(x / scale) unless t lies that close to k + 0.5; inside a far wider guard band the exact
//     division decides;
//   * adding 1.5 * 2^23 rounds to an integer (half to even) and leaves it in the low mantissa bits of the sum.
// Bit-identical to quantize_code.
__device__ __forceinline__ uint32_t quantize_code_fast(float x, float scale, float rscale) {
  const float kMagic = 12582912.f;                               // 1.5 * 2^23
  float t = fminf(fmaxf(x * rscale, -4.f), 4.f);
  float big = t + kMagic;
  const float q = big - kMagic;
  if (fabsf(fabsf(t - q) - 0.5f) < 1e-4f) {
    t = fminf(fmaxf(__fdiv_rn(x, scale), -4.f), 4.f);
    big = t + kMagic;
  }
  const int level = static_cast<int>(__float_as_uint(big) - 0x4B400000u) + 1;   // rint(x / scale) + 1
  return static_cast<uint32_t>(min(max(level, 0), 3));
}

// w: float32 [K, ld_w]; w_packed: uint8 [N, K/4]; scale_f32 / scale_f16: [K/G, N] (either may be null).
// G % 4 == 0, K % G == 0.  grid = (ceil(N / 128), K / G).
//
// One CTA = 128 consecutive output features x one scale group.  The group's tile of W (G rows x 128 floats) is
// brought into shared memory ONCE with 16-byte loads that are all in flight together (row-contiguous, so coalesced),
// in slabs of kPrepSlab rows; four threads then own one feature (a quarter of the slab's rows each): they scan their part
// of the column for the maximum and, once the scale is known, quantise and pack it out of shared memory (consecutive
// threads read consecutive words: no bank conflicts) and write 16-byte pieces of the feature's packed row.  Groups up to kPrepSlab rows (the usual 128) are
// read from HBM exactly once; longer groups re-read their slabs for the second pass.
constexpr int kPrepSlab = 128;
constexpr int kPrepParts = 4;             // threads per feature: each takes a quarter of a slab's rows
constexpr int kPrepCtaThreads = kPrepParts * kPrepThreads;

__global__ void __launch_bounds__(kPrepCtaThreads)
quantize_pack_weight_kernel(const float* __restrict__ w, long long ld_w, int K, int N, int G,
                            uint8_t* __restrict__ w_packed, float* __restrict__ scale_f32,
                            __half* __restrict__ scale_f16) {
  extern __shared__ float tile[];                 // [kPrepSlab][128]
  __shared__ float part_max[kPrepParts][kPrepThreads];
  const int f = threadIdx.x & (kPrepThreads - 1);  // feature within the tile
  const int part = threadIdx.x >> 7;               // which quarter of the rows
  const int n0 = blockIdx.x * kPrepThreads;
  const int n = n0 + f;
  const int g = blockIdx.y;
  const int cols = min(kPrepThreads, N - n0);
  const float* base = w + static_cast<long long>(g) * G * ld_w + n0;
  const bool vec_in = (cols == kPrepThreads) && ((ld_w & 3) == 0) && ((reinterpret_cast<uintptr_t>(base) & 15) == 0);

  auto load_slab = [&](int k0, int rows) {
    if (vec_in) {
      // 32 float4 per row; thread t takes float4 (t & 31) of rows (t >> 5), (t >> 5) + 16, ...
      const int c4 = threadIdx.x & 31;
      for (int r = threadIdx.x >> 5; r < rows; r += kPrepCtaThreads / 32)
        reinterpret_cast<float4*>(tile + r * kPrepThreads)[c4] =
            *reinterpret_cast<const float4*>(base + static_cast<long long>(k0 + r) * ld_w + 4 * c4);
    } else {
      for (int r = part; r < rows; r += kPrepParts)
        if (f < cols) tile[r * kPrepThreads + f] = base[static_cast<long long>(k0 + r) * ld_w + f];
    }
  };
  // rows [r_lo, r_hi) of a slab of `rows` rows belong to this thread: quarters when they are whole 32-row pieces
  auto my_rows = [&](int rows, int& r_lo, int& r_hi) {
    if ((rows % (32 * kPrepParts)) == 0) { r_lo = part * (rows / kPrepParts); r_hi = r_lo + rows / kPrepParts; }
    else { r_lo = 0; r_hi = part == 0 ? rows : 0; }
  };

  // pass 1: the column maxima
  float amax = 0.0f;
  for (int k0 = 0; k0 < G; k0 += kPrepSlab) {
    const int rows = min(kPrepSlab, G - k0);
    if (k0 > 0) __syncthreads();
    load_slab(k0, rows);
    __syncthreads();
    int r_lo, r_hi;
    my_rows(rows, r_lo, r_hi);
    if (f < cols) {
#pragma unroll 8
      for (int r = r_lo; r < r_hi; ++r) amax = fmaxf(amax, fabsf(tile[r * kPrepThreads + f]));
    }
  }
  part_max[part][f] = amax;
  __syncthreads();
#pragma unroll
  for (int q = 0; q < kPrepParts; ++q) amax = fmaxf(amax, part_max[q][f]);
  const float scale = __fdiv_rn(fmaxf(amax, 1e-9f), 1.5f);
  const float rscale = __fdiv_rn(1.0f, scale);
  if (part == 0 && f < cols) {
    if (scale_f32) scale_f32[static_cast<long long>(g) * N + n] = scale;
    if (scale_f16) scale_f16[static_cast<long long>(g) * N + n] = __float2half_rn(scale);
  }

  // pass 2: quantise and pack (the slab in shared memory is the group itself when G <= kPrepSlab)
  uint8_t* dst = w_packed + static_cast<long long>(n) * (K / 4) + static_cast<long long>(g) * (G / 4);
  for (int k0 = 0; k0 < G; k0 += kPrepSlab) {
    const int rows = min(kPrepSlab, G - k0);
    if (G > kPrepSlab) {
      __syncthreads();
      load_slab(k0, rows);
      __syncthreads();
    }
    int r_lo, r_hi;
    my_rows(rows, r_lo, r_hi);
    if (f >= cols || r_lo >= r_hi) continue;
    const float* colp = tile + f;
    uint8_t* d = dst + k0 / 4;
    const bool vec_out = ((r_hi - r_lo) % 32) == 0 && ((reinterpret_cast<uintptr_t>(d + r_lo / 4) & 7) == 0);
    if (vec_out) {
      for (int r0 = r_lo; r0 < r_hi; r0 += 32) {          // 32 codes -> 8 bytes
        uint32_t words[2];
#pragma unroll
        for (int wd = 0; wd < 2; ++wd) {
          uint32_t word = 0;
#pragma unroll
          for (int b = 0; b < 4; ++b) {             // byte b of the word: codes r0 + 16 wd + 4 b .. + 3
            uint32_t byte = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j)
              byte = (byte << 2) | quantize_code_fast(colp[(r0 + 16 * wd + 4 * b + j) * kPrepThreads], scale, rscale);
            word |= byte << (8 * b);
          }
          words[wd] = word;
        }
        *reinterpret_cast<uint2*>(d + r0 / 4) = make_uint2(words[0], words[1]);
      }
    } else {
      for (int r0 = r_lo; r0 < r_hi; r0 += 4) {
        uint32_t byte = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) byte = (byte << 2) | quantize_code_fast(colp[(r0 + j) * kPrepThreads], scale, rscale);
        d[r0 / 4] = static_cast<uint8_t>(byte);
      }
    }
  }
}

}  // namespace sk
