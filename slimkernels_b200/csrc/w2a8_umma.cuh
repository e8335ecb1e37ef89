// The W2A8 GEMM kernel for sm_100a.
//
// Stages (one CTA computes a tile of 128 output features x BLOCK_M tokens over a K range):
//   1. a producer thread brings, per 128-wide K block, one 4 KiB block of tiled 2-bit weights (bulk TMA copy)
//      and one BLOCK_M x 128 int8 activation tile (tensor-map TMA, 128-byte swizzle) into a ring of shared
//      memory stages guarded by mbarriers;
//   2. four expander warps turn the 2-bit codes into int8 bytes (code - zero_point), written straight into
//      the 128-byte-swizzled K-major layout the tensor core reads;
//   3. one thread issues tcgen05.mma kind::i8 (128 x BLOCK_M x 32 per instruction): the weights are the
//      "A"/M operand, the tokens the "B"/N operand, int32 accumulators live in tensor memory, one fresh
//      accumulator buffer per scale group (two buffers, so the next group accumulates while this one drains);
//   4. four epilogue warps read each finished group from tensor memory (lane = output feature, column =
//      token), convert to fp32, multiply by that feature's group scale (a per-thread scalar) and accumulate;
//      at the end the per-token activation scale is applied, the tile is transposed through shared memory
//      and written with 16-byte coalesced stores.
// With SPLIT_K > 1 the CTAs of one thread-block cluster split the groups of a tile and reduce their fp32
// accumulators through distributed shared memory in a fixed order (deterministic, no global scratch).
//
// This replaces the reference's gemm_device (slimkernels/cute/gemm/wgmma_sm90_W2A8.cu:165-424) and its
// in-register unpack + wgmma atom (slimkernels/cute/atom/mma_sm90_gmma.hpp:27-149); it shares no code with them.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ptx_sm100.cuh"

namespace sk {

constexpr int kTileN = 128;          // output features per CTA tile (MMA M)
constexpr int kBlockK = 128;         // K codes per pipeline stage (= one 128-byte swizzle row of int8)
constexpr int kStepK = 32;           // K per tcgen05.mma kind::i8
constexpr int kWpBytes = kTileN * kBlockK / 4;   // 4096: tiled 2-bit block
constexpr int kWxBytes = kTileN * kBlockK;       // 16384: expanded int8 block
constexpr int kNumThreads = 320;     // warps 0-3 epilogue, 4-7 expander, 8 producer, 9 MMA issuer
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // every mbarrier wait gives up after 2 s

// device status codes: role * 16 + barrier kind
enum : int {
  kStProducerEmpty = 0x11,
  kStExpanderFull = 0x21, kStExpanderEmpty = 0x22,
  kStMmaLdFull = 0x31, kStMmaExFull = 0x32, kStMmaAccEmpty = 0x33,
  kStEpilogueAccFull = 0x41,
  kStDrain = 0x51
};

struct GemmParams {
  const uint8_t* w_tiled;     // [n_tiles][k_blocks][4096]
  const __half* w_scale;      // [groups, N]
  const float* x_scale;       // [M]
  void* out;                  // [M, ld_out] half or bf16
  int32_t* partials;          // [groups, M, N] (debug mode) or nullptr
  int* status;                // device status word
  long long ld_out;
  int M, N, K;
  int k_blocks;               // ceil(K / 128)
  int k_steps;                // K / 32
  int steps_per_group;        // G / 32
  int groups;                 // K / G
  int zero_point;
  int out_bf16;
};

template <int BLOCK_M, int LSTAGES, int ESTAGES>
struct SmemLayout {
  static constexpr int kXBytes = BLOCK_M * kBlockK;
  static constexpr int kOffX = 0;
  static constexpr int kOffWx = kOffX + LSTAGES * kXBytes;
  static constexpr int kOffWp = kOffWx + ESTAGES * kWxBytes;
  static constexpr int kOffOut = kOffWp + LSTAGES * kWpBytes;
  static constexpr int kOutBytes = BLOCK_M * kTileN * 4;          // fp32 reduction tile or fp16/bf16 staging
  static constexpr int kOffBar = kOffOut + kOutBytes;
  static constexpr int kNumBars = 2 * LSTAGES + 2 * ESTAGES + 4;
  static constexpr int kOffMisc = kOffBar + kNumBars * 8;
  static constexpr int kTotal = kOffMisc + 16;
  static constexpr int kDynamicBytes = kTotal + 1024;             // slack for 1024-byte alignment of the base
};

struct WaitCtx {
  volatile int* abort_flag;  // shared memory
  int* status;               // global
};

// Bounded wait.  Returns false if the limit expired here or in any other thread of the CTA.
__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity, const WaitCtx& ctx, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*ctx.abort_flag) return false;
    if (globaltimer_ns() - t0 > kWaitLimitNs) {
      *ctx.abort_flag = 1;
      atomicCAS(ctx.status, 0, code);
      return false;
    }
  }
}

// 16 two-bit codes held in `w` as sum_{j,b} code[4j+b] << (8b + 2j)  ->  16 int8 bytes (code - zp), memory order.
__device__ __forceinline__ uint4 expand16(uint32_t w, uint32_t zp_bytes) {
  uint4 o;
  o.x = w & 0x03030303u;
  o.y = (w >> 2) & 0x03030303u;
  o.z = (w >> 4) & 0x03030303u;
  o.w = (w >> 6) & 0x03030303u;
  // per-byte (c - zp) without borrows across bytes: set bit 7, subtract, flip bit 7 back
  o.x = ((o.x | 0x80808080u) - zp_bytes) ^ 0x80808080u;
  o.y = ((o.y | 0x80808080u) - zp_bytes) ^ 0x80808080u;
  o.z = ((o.z | 0x80808080u) - zp_bytes) ^ 0x80808080u;
  o.w = ((o.w | 0x80808080u) - zp_bytes) ^ 0x80808080u;
  return o;
}

template <int BLOCK_M, int LSTAGES, int ESTAGES, bool DUMP>
__global__ void __launch_bounds__(kNumThreads, (BLOCK_M <= 32 ? 2 : 1))
w2a8_umma_kernel(const __grid_constant__ CUtensorMap tmap_x, const GemmParams p) {
  using L = SmemLayout<BLOCK_M, LSTAGES, ESTAGES>;
  constexpr int kChunk = (BLOCK_M >= 32) ? 32 : 16;      // TMEM columns per tcgen05.ld
  constexpr int kNumChunks = BLOCK_M / kChunk;
  constexpr uint32_t kTmemCols = (2 * BLOCK_M < 32) ? 32 : 2 * BLOCK_M;   // power of two >= 32
  constexpr uint32_t kStageTxBytes = kWpBytes + L::kXBytes;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + L::kOffBar;
  auto bar_ld_full = [&](int i) { return bar_base + 8u * i; };
  auto bar_ld_empty = [&](int i) { return bar_base + 8u * (LSTAGES + i); };
  auto bar_ex_full = [&](int i) { return bar_base + 8u * (2 * LSTAGES + i); };
  auto bar_ex_empty = [&](int i) { return bar_base + 8u * (2 * LSTAGES + ESTAGES + i); };
  auto bar_acc_full = [&](int i) { return bar_base + 8u * (2 * LSTAGES + 2 * ESTAGES + i); };
  auto bar_acc_empty = [&](int i) { return bar_base + 8u * (2 * LSTAGES + 2 * ESTAGES + 2 + i); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + L::kOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kOffMisc + 4);
  const WaitCtx ctx{abort_flag, p.status};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_tile = blockIdx.x;
  const int m_tile = blockIdx.y;
  const int split = blockIdx.z;
  const int num_splits = gridDim.z;
  const int n0 = n_tile * kTileN;
  const int m0 = m_tile * BLOCK_M;

  // K range of this CTA, in whole scale groups.
  const int groups_per_split = (p.groups + num_splits - 1) / num_splits;
  const int g_begin = min(split * groups_per_split, p.groups);
  const int g_end = min(g_begin + groups_per_split, p.groups);
  const int ks_begin = g_begin * p.steps_per_group;
  const int ks_end = g_end * p.steps_per_group;
  const int kb_begin = ks_begin / 4;
  const int kb_end = (ks_end + 3) / 4;

  // ---------------------------------------------------------------- set-up
  if (threadIdx.x == 0) {
    for (int i = 0; i < LSTAGES; ++i) { mbar_init(bar_ld_full(i), 1); mbar_init(bar_ld_empty(i), 1 + 128); }
    for (int i = 0; i < ESTAGES; ++i) { mbar_init(bar_ex_full(i), 128); mbar_init(bar_ex_empty(i), 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(bar_acc_full(i), 1); mbar_init(bar_acc_empty(i), 128); }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 8 && lane == 0) prefetch_tensormap(&tmap_x);
  if (warp == 9) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
    tmem_relinquish();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // fp32 accumulators of the epilogue threads (one output feature x BLOCK_M tokens each)
  float acc[BLOCK_M];
#pragma unroll
  for (int j = 0; j < BLOCK_M; ++j) acc[j] = 0.f;

  if (warp == 8) {
    // ============================================================ producer
    if (lane == 0) {
      const uint8_t* wsrc = p.w_tiled + (static_cast<size_t>(n_tile) * p.k_blocks + kb_begin) * kWpBytes;
      int issued = 0;
      bool ok = true;
      for (int kb = kb_begin; kb < kb_end && ok; ++kb, ++issued) {
        const int l = issued % LSTAGES;
        const uint32_t ph = (issued / LSTAGES) & 1;
        ok = wait_bounded(bar_ld_empty(l), ph ^ 1, ctx, kStProducerEmpty);
        if (!ok) break;
        mbar_arrive_expect_tx(bar_ld_full(l), kStageTxBytes);
        bulk_load_1d(smem_base + L::kOffWp + l * kWpBytes, wsrc + static_cast<size_t>(issued) * kWpBytes, kWpBytes,
                     bar_ld_full(l));
        tma_load_2d(smem_base + L::kOffX + l * L::kXBytes, &tmap_x, kb * kBlockK, m0, bar_ld_full(l));
      }
      if (!ok) {
        // Gave up: wait (bounded) until every copy this thread started has landed, so that none is in
        // flight into this CTA's shared memory when the CTA exits.
        const uint64_t t0 = globaltimer_ns();
        const int first = issued > LSTAGES ? issued - LSTAGES : 0;
        for (int i = first; i < issued; ++i) {
          const int l = i % LSTAGES;
          const uint32_t ph = (i / LSTAGES) & 1;
          while (!mbar_try_wait(bar_ld_full(l), ph)) {
            if (globaltimer_ns() - t0 > kWaitLimitNs) { atomicCAS(p.status, 0, kStDrain); break; }
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 9) {
    // ============================================================ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_i8(kTileN, BLOCK_M, /*a_signed=*/true, /*b_signed=*/true);
      int it = 0;      // k-blocks consumed
      int gcount = 0;  // groups started
      bool ok = true;
      for (int kb = kb_begin; kb < kb_end && ok; ++kb, ++it) {
        const int l = it % LSTAGES, e = it % ESTAGES;
        ok = wait_bounded(bar_ld_full(l), (it / LSTAGES) & 1, ctx, kStMmaLdFull) &&
             wait_bounded(bar_ex_full(e), (it / ESTAGES) & 1, ctx, kStMmaExFull);
        if (!ok) break;
        tcgen05_fence_after_sync();
        const uint64_t a_desc = make_kmajor_sw128_desc(smem_base + L::kOffWx + e * kWxBytes);
        const uint64_t b_desc = make_kmajor_sw128_desc(smem_base + L::kOffX + l * L::kXBytes);
#pragma unroll
        for (int s = 0; s < 4; ++s) {
          const int ks = kb * 4 + s;
          if (ks < ks_begin || ks >= ks_end) continue;
          const int pos = ks % p.steps_per_group;
          const int a = gcount & 1;
          if (pos == 0) {
            ok = wait_bounded(bar_acc_empty(a), ((gcount >> 1) & 1) ^ 1, ctx, kStMmaAccEmpty);
            if (!ok) break;
            tcgen05_fence_after_sync();
          }
          // advance 32 bytes along K inside the 128-byte swizzle row: +2 in the (address >> 4) field
          umma_i8(tmem_base + a * BLOCK_M, a_desc + 2 * s, b_desc + 2 * s, idesc, pos != 0);
          if (pos == p.steps_per_group - 1) {
            umma_commit(bar_acc_full(a));
            ++gcount;
          }
        }
        if (!ok) break;
        umma_commit(bar_ld_empty(l));
        umma_commit(bar_ex_empty(e));
      }
    }
    __syncwarp();
  } else if (warp >= 4) {
    // ============================================================ expanders (128 threads, one weight row each)
    const int row = threadIdx.x - 128;
    const uint32_t zp_bytes = 0x01010101u * static_cast<uint32_t>(p.zero_point);
    int it = 0;
    for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
      const int l = it % LSTAGES, e = it % ESTAGES;
      if (!wait_bounded(bar_ld_full(l), (it / LSTAGES) & 1, ctx, kStExpanderFull)) break;
      const uint8_t* wp = smem + L::kOffWp + l * kWpBytes;
      const uint4 lo = *reinterpret_cast<const uint4*>(wp + row * 16);          // codes   0..63 of this row
      const uint4 hi = *reinterpret_cast<const uint4*>(wp + 2048 + row * 16);   // codes 64..127
      mbar_arrive(bar_ld_empty(l));
      if (!wait_bounded(bar_ex_empty(e), ((it / ESTAGES) & 1) ^ 1, ctx, kStExpanderEmpty)) break;
      uint8_t* wx = smem + L::kOffWx + e * kWxBytes + row * 128;
      const int sw = row & 7;
      const uint32_t words[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *reinterpret_cast<uint4*>(wx + ((c ^ sw) << 4)) = expand16(words[c], zp_bytes);
      fence_proxy_async_smem();   // make the generic-proxy stores visible to the tensor core's async proxy
      mbar_arrive(bar_ex_full(e));
    }
  } else {
    // ============================================================ epilogue (warp w owns TMEM lanes 32w..32w+31)
    const int row = threadIdx.x;                 // output feature within the tile == TMEM lane
    const int n = n0 + row;
    const bool n_ok = n < p.N;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    float s_next = (n_ok && g_begin < g_end) ? __half2float(p.w_scale[static_cast<size_t>(g_begin) * p.N + n]) : 0.f;
    int gc = 0;
    for (int g = g_begin; g < g_end; ++g, ++gc) {
      const float s = s_next;
      if (g + 1 < g_end && n_ok) s_next = __half2float(p.w_scale[static_cast<size_t>(g + 1) * p.N + n]);
      const int a = gc & 1;
      if (!wait_bounded(bar_acc_full(a), (gc >> 1) & 1, ctx, kStEpilogueAccFull)) break;
      tcgen05_fence_after_sync();
#pragma unroll
      for (int c = 0; c < kNumChunks; ++c) {
        uint32_t v[kChunk];
        if constexpr (kChunk == 32) tmem_ld_32x32(lane_addr + a * BLOCK_M + c * kChunk, v);
        else tmem_ld_32x16(lane_addr + a * BLOCK_M + c * kChunk, v);
        tmem_ld_wait();
        if (c == kNumChunks - 1) {   // accumulator buffer fully read: hand it back to the MMA issuer
          tcgen05_fence_before_sync();
          mbar_arrive(bar_acc_empty(a));
        }
        if constexpr (DUMP) {
          if (n_ok) {
#pragma unroll
            for (int j = 0; j < kChunk; ++j) {
              const int m = m0 + c * kChunk + j;
              if (m < p.M) p.partials[(static_cast<size_t>(g) * p.M + m) * p.N + n] = static_cast<int32_t>(v[j]);
            }
          }
        }
#pragma unroll
        for (int j = 0; j < kChunk; ++j)
          acc[c * kChunk + j] = fmaf(s, static_cast<float>(static_cast<int32_t>(v[j])), acc[c * kChunk + j]);
      }
    }
  }

  // ---------------------------------------------------------------- output
  if constexpr (!DUMP) {
    if (num_splits == 1) {
      if (warp < 4) {
        const int row = threadIdx.x;
        // stage the tile transposed: [token][feature] in the output dtype
        uint16_t* st = reinterpret_cast<uint16_t*>(smem + L::kOffOut);
#pragma unroll
        for (int j = 0; j < BLOCK_M; ++j) {
          const int m = m0 + j;
          const float xs = (m < p.M) ? __ldg(p.x_scale + m) : 0.f;
          const float y = acc[j] * xs;
          st[j * kTileN + row] = p.out_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(y))
                                            : __half_as_ushort(__float2half_rn(y));
        }
        named_barrier_sync(1, 128);
        uint16_t* outp = reinterpret_cast<uint16_t*>(p.out);
        const bool vec_ok = (n0 + kTileN <= p.N) && (p.ld_out % 8 == 0) &&
                            ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
        if (vec_ok) {
          // 16 threads x 16 bytes cover one 256-byte row of the tile
          for (int idx = threadIdx.x; idx < BLOCK_M * 16; idx += 128) {
            const int j = idx >> 4, ch = idx & 15;
            const int m = m0 + j;
            if (m < p.M)
              *reinterpret_cast<uint4*>(outp + static_cast<size_t>(m) * p.ld_out + n0 + ch * 8) =
                  *reinterpret_cast<const uint4*>(st + j * kTileN + ch * 8);
          }
        } else {
          for (int idx = threadIdx.x; idx < BLOCK_M * kTileN; idx += 128) {
            const int j = idx >> 7, r = idx & 127;
            const int m = m0 + j;
            if (m < p.M && n0 + r < p.N) outp[static_cast<size_t>(m) * p.ld_out + n0 + r] = st[j * kTileN + r];
          }
        }
      }
    } else {
      // split-K: fixed-order reduction over the cluster through distributed shared memory
      float* red = reinterpret_cast<float*>(smem + L::kOffOut);
      if (warp < 4) {
#pragma unroll
        for (int j = 0; j < BLOCK_M; ++j) red[j * kTileN + threadIdx.x] = acc[j];
      }
      cluster_sync_all();
      if (warp < 4) {
        const uint32_t my_rank = cluster_ctarank();
        const int row = threadIdx.x;
        const int n = n0 + row;
        uint16_t* outp = reinterpret_cast<uint16_t*>(p.out);
        for (int j = static_cast<int>(my_rank); j < BLOCK_M; j += num_splits) {
          const int m = m0 + j;
          if (m >= p.M) break;
          const uint32_t local = smem_u32(red + j * kTileN + row);
          float sum = 0.f;
          for (int r = 0; r < num_splits; ++r) sum += ld_dsmem_f32(map_to_cta(local, r));
          const float y = sum * __ldg(p.x_scale + m);
          if (n < p.N)
            outp[static_cast<size_t>(m) * p.ld_out + n] = p.out_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(y))
                                                                     : __half_as_ushort(__float2half_rn(y));
        }
      }
      cluster_sync_all();   // peers may still be reading this CTA's shared memory until here
    }
  }

  // ---------------------------------------------------------------- teardown
  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 9) {
    tcgen05_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace sk
