// Activation-side kernels of the W2A8 MLP block: per-token symmetric int8 quantisation and the fused
// SiLU(gate) * up -> int8 re-quantisation between the gate+up and down projections.
// The reference has no activation quantiser (its prototype feeds pre-made e4m3 tensors,
// slimkernels/cute/gemm/wgmma_sm90_W2A8.cu:541-552); the definition here is this library's:
//     s[m] = max_k |x[m,k]| / 127   (1.0 for an all-zero row),   q[m,k] = clamp(rint(x[m,k] / s[m]), -127, 127)
// Both kernels are HBM-bound row passes with 16-byte loads; the row is kept in registers between the max pass and the
// quantise pass (one CTA per row for the plain quantiser, a cluster of CTAs per row for the SiLU one).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sk {

constexpr int kActThreads = 256;

// Programmatic dependent launch (both are no-ops for a kernel launched without the attribute): the next kernel in the
// stream may start its own set-up now -- the decode GEMM that follows a quantiser uses that to stream its first
// weights --, and this kernel's inputs, which the previous kernel wrote, are read only after that kernel is complete.
__device__ __forceinline__ void act_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void act_wait_for_inputs() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

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

// The same integer without the division, the rounding instruction or the float -> int conversion (an IEEE division
// is ~10 instructions, and rint / cvt issue at an eighth of the FMA rate; these kernels do one of each per element):
//   * t = x * r with r = 1 / s differs from the rounded quotient x / s by a few units in the last place (< 3e-5 at
//     |t| <= 128), so rint(t) == rint(x / s) unless t lies within that distance of k + 0.5; inside a far wider guard
//     band (1e-3) the exact division decides, so the result is bit-identical to quantize_one;
//   * adding 1.5 * 2^23 rounds t to an integer (round half to even, the FADD's own rounding) and leaves that integer,
//     in two's complement, in the low mantissa bits of the sum.
// Returns the integer's low 8 bits (what the packed int8 row wants).
__device__ __forceinline__ uint32_t quantize_one_fast(float x, float s, float r) {
  const float kMagic = 12582912.f;                               // 1.5 * 2^23
  float t = fminf(fmaxf(x * r, -127.f), 127.f);
  float big = t + kMagic;
  const float q = big - kMagic;
  if (fabsf(t - q) > 0.499f) {                                   // (|t - q| <= 0.5) rare: decided by the exact quotient
    t = fminf(fmaxf(x / s, -127.f), 127.f);
    big = t + kMagic;
  }
  return __float_as_uint(big) & 0xffu;
}

// x fp16 [M, ld_x] -> x_q int8 [M, ld_q], x_scale fp32 [M].  K % 8 == 0, rows 16-byte aligned.
// Each thread keeps its 8-element vectors of the row in registers (up to kMaxVec of them); longer rows are re-read.
template <int kMaxVec>
__global__ void __launch_bounds__(kActThreads)
quantize_activation_kernel(const __half* __restrict__ x, long long ld_x, int8_t* __restrict__ x_q, long long ld_q,
                           float* __restrict__ x_scale, int K) {
  __shared__ float red[kActThreads / 32];
  act_launch_dependents();
  act_wait_for_inputs();
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
  const float r = 1.f / s;
  if (threadIdx.x == 0) x_scale[m] = s;
  uint2* qrow = reinterpret_cast<uint2*>(x_q + m * ld_q);
  auto emit = [&](int v, const uint4& t) {
    const __half2* h = reinterpret_cast<const __half2*>(&t);
    uint32_t w[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(h[j]);
      const uint32_t a = quantize_one_fast(f.x, s, r);
      const uint32_t b = quantize_one_fast(f.y, s, r);
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
// h_q int8 [M, ld_q], h_scale fp32 [M].  I % 8 == 0.
// SiLU(g) * u = g * u / (1 + exp(-g)) in fp32.  The exponential and the reciprocal are the hardware approximations
// (ex2.approx, rcp.approx: about two units in the last place each); an IEEE division and expf cost four times the
// instructions and the result feeds an 8-bit quantiser.
__device__ __forceinline__ float silu_mul(float g, float u) {
  return __fdividef(g * u, 1.f + __expf(-g));
}

// One pass over HBM for rows of any practical length: a row is split over the CTAs of a thread-block cluster (1, 2, 4
// or 8 CTAs along x), every thread keeps the fp32 values of its kClusterVecs 8-element vectors in registers, the row
// maximum is exchanged through distributed shared memory (each CTA stores its partial maximum into every CTA of the
// cluster, one cluster barrier), and the quantised row is written from the registers: the gate / up vectors are read
// once and SiLU is evaluated once.  Rows up to 8 * 256 * kClusterVecs * cluster size elements.
constexpr int kClusterVecs = 2;

// (eight CTAs per SM: 32 registers per thread instead of 40 cost a few spilled words and gain 13 % -- the kernel's
// phases -- load, SiLU, barriers, quantise, store -- overlap only across the CTAs of an SM)
__global__ void __launch_bounds__(kActThreads, 8)
silu_mul_quantize_cluster_kernel(const __half* __restrict__ gate_up, long long ld_gu, int8_t* __restrict__ h_q,
                                 long long ld_q, float* __restrict__ h_scale, int I) {
  __shared__ float red[kActThreads / 32];
  __shared__ float part[8];                     // partial maxima of the cluster's CTAs
  act_launch_dependents();
  act_wait_for_inputs();
  const long long m = blockIdx.y;
  const int csize = static_cast<int>(gridDim.x);   // the cluster spans the grid's x dimension
  const int crank = static_cast<int>(blockIdx.x);
  const uint4* g = reinterpret_cast<const uint4*>(gate_up + m * ld_gu);
  const uint4* u = reinterpret_cast<const uint4*>(gate_up + m * ld_gu + I);
  const int nvec = I / 8;
  const int per = (nvec + csize - 1) / csize;   // vectors of this CTA: [v0, v1)
  const int v0 = crank * per, v1 = min(nvec, v0 + per);
  float h[kClusterVecs][8];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < kClusterVecs; ++i) {
    const int v = v0 + threadIdx.x + i * kActThreads;
    if (v < v1) {
      const uint4 gv = g[v], uv = u[v];
      const __half2* gh = reinterpret_cast<const __half2*>(&gv);
      const __half2* uh = reinterpret_cast<const __half2*>(&uv);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 gf = __half22float2(gh[j]), uf = __half22float2(uh[j]);
        h[i][2 * j] = silu_mul(gf.x, uf.x);
        h[i][2 * j + 1] = silu_mul(gf.y, uf.y);
        amax = fmaxf(amax, fmaxf(fabsf(h[i][2 * j]), fabsf(h[i][2 * j + 1])));
      }
    }
  }
  amax = block_max(amax, red);
  if (csize > 1) {
    if (threadIdx.x < csize) {
      uint32_t remote;
      const uint32_t local = static_cast<uint32_t>(__cvta_generic_to_shared(&part[crank]));
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(threadIdx.x));
      asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(amax) : "memory");
    }
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    float a = 0.f;
    for (int c = 0; c < csize; ++c) a = fmaxf(a, part[c]);
    amax = a;
  }
  const float s = amax > 0.f ? amax / 127.f : 1.f;
  const float r = 1.f / s;
  if (threadIdx.x == 0 && crank == 0) h_scale[m] = s;
  uint2* qrow = reinterpret_cast<uint2*>(h_q + m * ld_q);
#pragma unroll
  for (int i = 0; i < kClusterVecs; ++i) {
    const int v = v0 + threadIdx.x + i * kActThreads;
    if (v < v1) {
      uint32_t w[2] = {0u, 0u};
#pragma unroll
      for (int j = 0; j < 8; ++j)
        w[j >> 2] |= quantize_one_fast(h[i][j], s, r) << (8 * (j & 3));
      qrow[v] = make_uint2(w[0], w[1]);
    }
  }
}

// Same result for rows longer than the cluster kernel takes, where the fp32 row in shared memory (4 * I bytes) would leave one CTA per SM: the row is
// read twice instead (the second pass is an L2 hit) and SiLU(gate) * up is recomputed, which gives the identical
// fp32 values; no dynamic shared memory, so eight CTAs fit an SM.
__global__ void __launch_bounds__(kActThreads)
silu_mul_quantize_twopass_kernel(const __half* __restrict__ gate_up, long long ld_gu, int8_t* __restrict__ h_q,
                                 long long ld_q, float* __restrict__ h_scale, int I) {
  __shared__ float red[kActThreads / 32];
  act_launch_dependents();
  act_wait_for_inputs();
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
      h[2 * j] = silu_mul(gf.x, uf.x);
      h[2 * j + 1] = silu_mul(gf.y, uf.y);
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


// Sum of n_blocks row blocks [rows][N] (16-bit floats, block pitch `block_stride` elements, row pitch ld) in fp32 in
// block order, rounded once to the same 16-bit type: the add half of the reduce-scatter of K-sharded partial sums.
// 8 elements (16 bytes) per thread; N % 8 == 0.
template <bool BF16>
__global__ void sum_row_blocks_kernel(const uint16_t* __restrict__ blocks, long long block_stride, long long ld,
                                      int n_blocks, long long rows, int N, uint16_t* __restrict__ out, long long ld_out) {
  const int vec_per_row = N / 8;
  const long long total = rows * vec_per_row;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = static_cast<int>(i - r * vec_per_row) * 8;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int b = 0; b < n_blocks; ++b) {
      const uint4 v = *reinterpret_cast<const uint4*>(blocks + b * block_stride + r * ld + c);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float lo, hi;
        if constexpr (BF16) {
          lo = __uint_as_float(w[j] << 16);
          hi = __uint_as_float(w[j] & 0xffff0000u);
        } else {
          const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
          lo = f.x; hi = f.y;
        }
        acc[2 * j] += lo;
        acc[2 * j + 1] += hi;
      }
    }
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if constexpr (BF16) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        o[j] = *reinterpret_cast<const uint32_t*>(&h);
      } else {
        const __half2 h = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
        o[j] = *reinterpret_cast<const uint32_t*>(&h);
      }
    }
    *reinterpret_cast<uint4*>(out + r * ld_out + c) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

}  // namespace sk
