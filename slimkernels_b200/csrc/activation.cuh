// Activation-side kernels of the W2A8 MLP block: per-token symmetric int8 quantisation and the fused
// SiLU(gate) * up -> int8 re-quantisation between the gate+up and down projections.
// The reference has no activation quantiser (its prototype feeds pre-made e4m3 tensors,
// slimkernels/cute/gemm/wgmma_sm90_W2A8.cu:541-552); the definition here is this library's:
//     s[m] = max_k |x[m,k]| / 127   (1.0 for an all-zero row),   q[m,k] = clamp(rint(x[m,k] / s[m]), -127, 127)
// Both kernels are HBM-bound row passes: one CTA per token row, 16-byte loads, the row is kept on chip between the
// max pass and the quantise pass (registers for the plain quantiser, shared memory for the SiLU one).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sk {

constexpr int kActThreads = 256;

__device__ __forceinline__ float block_max(float v, float* red /* [kActThreads / 32] */) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = (lane < kActThreads / 32) ? red[lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r = fmaxf(r, __shfl_xor_sync(0xffffffffu, r, o));
  __syncthreads();
  return r;
}

__device__ __forceinline__ int quantize_one(float x, float s) {
  const float q = rintf(x / s);                       // IEEE division, round half to even
  return static_cast<int>(fminf(fmaxf(q, -127.f), 127.f));
}

// x fp16 [M, ld_x] -> x_q int8 [M, ld_q], x_scale fp32 [M].  K % 8 == 0, rows 16-byte aligned.
// Each thread keeps its 8-element vectors of the row in registers (up to kMaxVec of them); longer rows are re-read.
template <int kMaxVec>
__global__ void __launch_bounds__(kActThreads)
quantize_activation_kernel(const __half* __restrict__ x, long long ld_x, int8_t* __restrict__ x_q, long long ld_q,
                           float* __restrict__ x_scale, int K) {
  __shared__ float red[kActThreads / 32];
  const long long m = blockIdx.x;
  const uint4* row = reinterpret_cast<const uint4*>(x + m * ld_x);
  const int nvec = K / 8;
  uint4 keep[kMaxVec];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int v = threadIdx.x + i * kActThreads;
    if (v < nvec) {
      keep[i] = row[v];
      const __half2* h = reinterpret_cast<const __half2*>(&keep[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h[j]);
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
    }
  }
  for (int v = threadIdx.x + kMaxVec * kActThreads; v < nvec; v += kActThreads) {   // rows longer than the cache
    const uint4 t = row[v];
    const __half2* h = reinterpret_cast<const __half2*>(&t);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(h[j]);
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  amax = block_max(amax, red);
  const float s = amax > 0.f ? amax / 127.f : 1.f;
  if (threadIdx.x == 0) x_scale[m] = s;
  uint2* qrow = reinterpret_cast<uint2*>(x_q + m * ld_q);
  auto emit = [&](int v, const uint4& t) {
    const __half2* h = reinterpret_cast<const __half2*>(&t);
    uint32_t w[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(h[j]);
      const uint32_t a = static_cast<uint32_t>(quantize_one(f.x, s)) & 0xffu;
      const uint32_t b = static_cast<uint32_t>(quantize_one(f.y, s)) & 0xffu;
      w[j >> 1] |= (a | (b << 8)) << (16 * (j & 1));
    }
    qrow[v] = make_uint2(w[0], w[1]);
  };
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int v = threadIdx.x + i * kActThreads;
    if (v < nvec) emit(v, keep[i]);
  }
  for (int v = threadIdx.x + kMaxVec * kActThreads; v < nvec; v += kActThreads) emit(v, row[v]);
}

// gate_up fp16 [M, ld_gu] with gate = columns [0, I), up = columns [I, 2I)  ->  h = SiLU(gate) * up (fp32),
// h_q int8 [M, ld_q], h_scale fp32 [M].  I % 8 == 0.  The fp32 row is kept in dynamic shared memory (4 * I bytes).
__global__ void __launch_bounds__(kActThreads)
silu_mul_quantize_kernel(const __half* __restrict__ gate_up, long long ld_gu, int8_t* __restrict__ h_q, long long ld_q,
                         float* __restrict__ h_scale, int I) {
  extern __shared__ float hrow[];
  __shared__ float red[kActThreads / 32];
  const long long m = blockIdx.x;
  const uint4* g = reinterpret_cast<const uint4*>(gate_up + m * ld_gu);
  const uint4* u = reinterpret_cast<const uint4*>(gate_up + m * ld_gu + I);
  const int nvec = I / 8;
  float amax = 0.f;
  for (int v = threadIdx.x; v < nvec; v += kActThreads) {
    const uint4 gv = g[v], uv = u[v];
    const __half2* gh = reinterpret_cast<const __half2*>(&gv);
    const __half2* uh = reinterpret_cast<const __half2*>(&uv);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 gf = __half22float2(gh[j]), uf = __half22float2(uh[j]);
      const float h0 = (gf.x / (1.f + expf(-gf.x))) * uf.x;
      const float h1 = (gf.y / (1.f + expf(-gf.y))) * uf.y;
      hrow[v * 8 + 2 * j] = h0;
      hrow[v * 8 + 2 * j + 1] = h1;
      amax = fmaxf(amax, fmaxf(fabsf(h0), fabsf(h1)));
    }
  }
  amax = block_max(amax, red);   // also orders the hrow writes before the reads below
  const float s = amax > 0.f ? amax / 127.f : 1.f;
  if (threadIdx.x == 0) h_scale[m] = s;
  uint2* qrow = reinterpret_cast<uint2*>(h_q + m * ld_q);
  for (int v = threadIdx.x; v < nvec; v += kActThreads) {
    uint32_t w[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 8; ++j)
      w[j >> 2] |= (static_cast<uint32_t>(quantize_one(hrow[v * 8 + j], s)) & 0xffu) << (8 * (j & 3));
    qrow[v] = make_uint2(w[0], w[1]);
  }
}

// Same result for long rows, where the fp32 row in shared memory (4 * I bytes) would leave one CTA per SM: the row is
// read twice instead (the second pass is an L2 hit) and SiLU(gate) * up is recomputed, which gives the identical
// fp32 values; no dynamic shared memory, so eight CTAs fit an SM.
__global__ void __launch_bounds__(kActThreads)
silu_mul_quantize_twopass_kernel(const __half* __restrict__ gate_up, long long ld_gu, int8_t* __restrict__ h_q,
                                 long long ld_q, float* __restrict__ h_scale, int I) {
  __shared__ float red[kActThreads / 32];
  const long long m = blockIdx.x;
  const uint4* g = reinterpret_cast<const uint4*>(gate_up + m * ld_gu);
  const uint4* u = reinterpret_cast<const uint4*>(gate_up + m * ld_gu + I);
  const int nvec = I / 8;
  auto silu_mul8 = [](const uint4& gv, const uint4& uv, float (&h)[8]) {
    const __half2* gh = reinterpret_cast<const __half2*>(&gv);
    const __half2* uh = reinterpret_cast<const __half2*>(&uv);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 gf = __half22float2(gh[j]), uf = __half22float2(uh[j]);
      h[2 * j] = (gf.x / (1.f + expf(-gf.x))) * uf.x;
      h[2 * j + 1] = (gf.y / (1.f + expf(-gf.y))) * uf.y;
    }
  };
  float amax = 0.f;
  for (int v = threadIdx.x; v < nvec; v += kActThreads) {
    float h[8];
    silu_mul8(g[v], u[v], h);
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(h[j]));
  }
  amax = block_max(amax, red);
  const float s = amax > 0.f ? amax / 127.f : 1.f;
  if (threadIdx.x == 0) h_scale[m] = s;
  uint2* qrow = reinterpret_cast<uint2*>(h_q + m * ld_q);
  for (int v = threadIdx.x; v < nvec; v += kActThreads) {
    float h[8];
    silu_mul8(g[v], u[v], h);
    uint32_t w[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 8; ++j)
      w[j >> 2] |= (static_cast<uint32_t>(quantize_one(h[j], s)) & 0xffu) << (8 * (j & 3));
    qrow[v] = make_uint2(w[0], w[1]);
  }
}

}  // namespace sk
