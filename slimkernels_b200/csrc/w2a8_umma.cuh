// The W2A8 GEMM kernel for sm_100a.
//
// One CTA computes a tile of 128 output features x BLOCK_M tokens over a range of scale groups:
//   1. a producer thread brings, per 128-wide K block, one 4 KiB block of tiled 2-bit weights (bulk TMA copy)
//      and one BLOCK_M x 128 int8 activation tile (tensor-map TMA, 128-byte swizzle) into a ring of shared
//      memory stages guarded by mbarriers;
//   2. one warpgroup of expander threads turns the 2-bit codes into int8 bytes (code - zero_point) with a
//      byte-permute look-up (prmt), written straight into the 128-byte-swizzled K-major layout the tensor
//      core reads;
//   3. one thread issues tcgen05.mma kind::i8 (128 x BLOCK_M x 32 per instruction): the weights are the
//      "A"/M operand, the tokens the "B"/N operand, int32 accumulators live in tensor memory, one accumulator
//      buffer per scale group (two buffers, so the next group accumulates while this one drains);
//   4. one or two epilogue warpgroups read each finished group from tensor memory (lane = output feature,
//      column = token), multiply by that feature's group scale (a per-thread scalar) and accumulate in fp32;
//      at the end the per-token activation scale is applied, the tile is transposed through shared memory
//      and written with 16-byte coalesced stores.
//
// Integer -> float without a conversion instruction: every accumulator buffer is pre-set to a positive bias B
// (2^15, or 2^16 when |code - zp| can reach 3) and the MMAs always accumulate, so a finished group holds
// D = B + P with 0 < D < 2^23.  Read as an IEEE float, those bits are the denormal D * 2^-149, exactly.  The
// epilogue therefore needs ONE fused multiply-add per value, acc += (s * 2^100) * asfloat(D); the bias term
// B * sum_g s is the same for every token of a thread and is removed with one subtraction per 16 groups.
// The exact partial sum P = D - B is what the debug entry point stores.
//
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
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // every mbarrier wait gives up after 2 s
constexpr int kBiasFlushGroups = 16;  // the bias term is subtracted from the accumulators this often

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
  int steps_per_group;        // G / 32
  int groups;                 // K / G
  int zero_point;
  int out_bf16;
};

template <int BLOCK_M, int EPI_WGS, int LSTAGES, int ESTAGES>
struct KernelTraits {
  static constexpr int kThreads = (EPI_WGS + 2) * 128;
  static constexpr int kEpiThreads = EPI_WGS * 128;
  static constexpr int kColsPerWg = BLOCK_M / EPI_WGS;           // accumulators per epilogue thread
  static constexpr int kChunk = (kColsPerWg >= 32 && kColsPerWg <= 64) ? 32 : 16;   // TMEM columns per tcgen05.ld
  static constexpr int kNumChunks = kColsPerWg / kChunk;
  static constexpr uint32_t kTmemCols = (2 * BLOCK_M < 32) ? 32 : 2 * BLOCK_M;   // power of two >= 32
  static constexpr int kXBytes = BLOCK_M * kBlockK;
  static constexpr int kOffX = 0;
  static constexpr int kOffWx = kOffX + LSTAGES * kXBytes;
  static constexpr int kOffWp = kOffWx + ESTAGES * kWxBytes;
  static constexpr int kOffBar = kOffWp + LSTAGES * kWpBytes;
  static constexpr int kNumBars = 2 * LSTAGES + 2 * ESTAGES + 4;
  static constexpr int kOffMisc = kOffBar + kNumBars * 8;
  static constexpr int kOffXs = kOffMisc + 16;                   // fp32 [BLOCK_M]: x_scale of the tile's tokens
  static constexpr int kTotal = kOffXs + BLOCK_M * 4;
  static constexpr int kDynamicBytes = kTotal + 1024;            // slack for 1024-byte alignment of the base
  // After the main loop the operand ring is dead and is reused for the output tile
  // (fp32 [BLOCK_M][128] for the split-K reduction, 16-bit [BLOCK_M][128] otherwise).
  static_assert(BLOCK_M * kTileN * 4 <= kOffBar, "output staging must fit in the operand ring");
  static_assert(kColsPerWg % kChunk == 0 && kNumChunks >= 1, "bad epilogue split");
  // Two epilogue warpgroups (512 threads, 128 registers each at launch): the epilogue warpgroups take registers
  // from the expander / control warpgroups.  2 * 128 * (kEpiRegs + kOtherRegs) == 65536.
  static constexpr bool kUseSetMaxNReg = (EPI_WGS == 2);
  static constexpr int kEpiRegs = kColsPerWg > 64 ? 192 : 160;
  static constexpr int kOtherRegs = 256 - kEpiRegs;
  // Two register sets for TMEM loads (load chunk c+1 while chunk c is consumed) only where registers allow.
  static constexpr bool kDoubleBuf = (kNumChunks > 1) && (EPI_WGS == 1);
  static constexpr int kMinBlocks = (BLOCK_M <= 32) ? 2 : 1;
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

// 16 two-bit codes held in `w` as  sum_{j,b} code[4j+b] << (4b + 2(j&1) + 16(j>>1))  ->  16 int8 bytes
// lut[code] in memory order; lut = the four bytes (0-zp, 1-zp, 2-zp, 3-zp).
__device__ __forceinline__ uint4 expand16(uint32_t w, uint32_t lut) {
  const uint32_t lo = w & 0x33333333u;          // low code of every nibble  (j even)
  const uint32_t hi = (w >> 2) & 0x33333333u;   // high code of every nibble (j odd)
  uint4 o;
  o.x = prmt(lut, lut, lo);
  o.y = prmt(lut, lut, hi);
  o.z = prmt(lut, lut, lo >> 16);
  o.w = prmt(lut, lut, hi >> 16);
  return o;
}

template <int BLOCK_M, int EPI_WGS, int LSTAGES, int ESTAGES, bool DUMP>
__global__ void __launch_bounds__((EPI_WGS + 2) * 128, (BLOCK_M <= 32 ? 2 : 1))
w2a8_umma_kernel(const __grid_constant__ CUtensorMap tmap_x, const GemmParams p) {
  using T = KernelTraits<BLOCK_M, EPI_WGS, LSTAGES, ESTAGES>;
  constexpr int kChunk = T::kChunk;
  constexpr int kNumChunks = T::kNumChunks;
  constexpr int kCols = T::kColsPerWg;
  constexpr uint32_t kStageTxBytes = kWpBytes + T::kXBytes;
  constexpr int kExpWarp0 = EPI_WGS * 4;        // first expander warp
  constexpr int kProducerWarp = kExpWarp0 + 4;
  constexpr int kMmaWarp = kProducerWarp + 1;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + T::kOffBar;
  auto bar_ld_full = [&](int i) { return bar_base + 8u * i; };
  auto bar_ld_empty = [&](int i) { return bar_base + 8u * (LSTAGES + i); };
  auto bar_ex_full = [&](int i) { return bar_base + 8u * (2 * LSTAGES + i); };
  auto bar_ex_empty = [&](int i) { return bar_base + 8u * (2 * LSTAGES + ESTAGES + i); };
  auto bar_acc_full = [&](int i) { return bar_base + 8u * (2 * LSTAGES + 2 * ESTAGES + i); };
  auto bar_acc_empty = [&](int i) { return bar_base + 8u * (2 * LSTAGES + 2 * ESTAGES + 2 + i); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + T::kOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + T::kOffMisc + 4);
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

  // |code - zp| <= 2 keeps |P| <= 128*127*2 < 2^15; zero points 0 and 3 need the next power of two.
  const uint32_t bias = (p.zero_point == 1 || p.zero_point == 2) ? 32768u : 65536u;

  // ---------------------------------------------------------------- set-up
  if (threadIdx.x == 0) {
    for (int i = 0; i < LSTAGES; ++i) { mbar_init(bar_ld_full(i), 1); mbar_init(bar_ld_empty(i), 1 + 128); }
    for (int i = 0; i < ESTAGES; ++i) { mbar_init(bar_ex_full(i), 128); mbar_init(bar_ex_empty(i), 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(bar_acc_full(i), 1); mbar_init(bar_acc_empty(i), T::kEpiThreads); }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == kProducerWarp && lane == 0) prefetch_tensormap(&tmap_x);
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), T::kTmemCols);
    tmem_relinquish();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp >= kExpWarp0) {
    if constexpr (T::kUseSetMaxNReg) setmaxnreg_dec<T::kOtherRegs>();
    if (warp == kProducerWarp) {
      // ============================================================ producer
      if (lane == 0) {
        const uint8_t* wsrc = p.w_tiled + (static_cast<size_t>(n_tile) * p.k_blocks + kb_begin) * kWpBytes;
        int issued = 0;
        bool ok = true;
        for (int kb = kb_begin; kb < kb_end; ++kb, ++issued) {
          const int l = issued % LSTAGES;
          const uint32_t ph = (issued / LSTAGES) & 1;
          ok = wait_bounded(bar_ld_empty(l), ph ^ 1, ctx, kStProducerEmpty);
          if (!ok) break;
          mbar_arrive_expect_tx(bar_ld_full(l), kStageTxBytes);
          bulk_load_1d(smem_base + T::kOffWp + l * kWpBytes, wsrc + static_cast<size_t>(issued) * kWpBytes,
                       kWpBytes, bar_ld_full(l));
          tma_load_2d(smem_base + T::kOffX + l * T::kXBytes, &tmap_x, kb * kBlockK, m0, bar_ld_full(l));
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
    } else if (warp == kMmaWarp) {
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
          const uint64_t a_desc = make_kmajor_sw128_desc(smem_base + T::kOffWx + e * kWxBytes);
          const uint64_t b_desc = make_kmajor_sw128_desc(smem_base + T::kOffX + l * T::kXBytes);
#pragma unroll
          for (int s = 0; s < 4; ++s) {
            const int ks = kb * 4 + s;
            if (ks < ks_begin || ks >= ks_end) continue;
            const int pos = ks % p.steps_per_group;
            const int a = gcount & 1;
            if (pos == 0) {
              // the epilogue pre-sets (and later re-sets) the buffer to the bias before releasing it
              ok = wait_bounded(bar_acc_empty(a), (gcount >> 1) & 1, ctx, kStMmaAccEmpty);
              if (!ok) break;
              tcgen05_fence_after_sync();
            }
            // advance 32 bytes along K inside the 128-byte swizzle row: +2 in the (address >> 4) field
            umma_i8(tmem_base + a * BLOCK_M, a_desc + 2 * s, b_desc + 2 * s, idesc, 1u);
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
    } else if (warp < kProducerWarp) {
      // ============================================================ expanders (128 threads, one weight row each)
      const int row = threadIdx.x - kExpWarp0 * 32;
      const int zp = p.zero_point;
      const uint32_t lut = (static_cast<uint32_t>(0 - zp) & 0xffu) | ((static_cast<uint32_t>(1 - zp) & 0xffu) << 8) |
                           ((static_cast<uint32_t>(2 - zp) & 0xffu) << 16) | ((static_cast<uint32_t>(3 - zp) & 0xffu) << 24);
      int it = 0;
      for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
        const int l = it % LSTAGES, e = it % ESTAGES;
        if (!wait_bounded(bar_ld_full(l), (it / LSTAGES) & 1, ctx, kStExpanderFull)) break;
        if (!wait_bounded(bar_ex_empty(e), ((it / ESTAGES) & 1) ^ 1, ctx, kStExpanderEmpty)) break;
        const uint8_t* wp = smem + T::kOffWp + l * kWpBytes + row * 16;
        uint8_t* wx = smem + T::kOffWx + e * kWxBytes + row * 128;
        const int sw = row & 7;
#pragma unroll
        for (int h = 0; h < 2; ++h) {     // codes 64h .. 64h+63 of this row: 16 bytes in, 64 bytes out
          const uint4 q = *reinterpret_cast<const uint4*>(wp + h * 2048);
          const uint32_t words[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (int c = 0; c < 4; ++c)
            *reinterpret_cast<uint4*>(wx + (((4 * h + c) ^ sw) << 4)) = expand16(words[c], lut);
          asm volatile("" ::: "memory");
        }
        mbar_arrive(bar_ld_empty(l));
        fence_proxy_async_smem();   // make the generic-proxy stores visible to the tensor core's async proxy
        mbar_arrive(bar_ex_full(e));
      }
    }
  } else {
    // ============================================================ epilogue
    // warp w: TMEM lanes 32 (w % 4) .. +31 (hardware rule), token columns of warpgroup w / 4
    if constexpr (T::kUseSetMaxNReg) setmaxnreg_inc<T::kEpiRegs>();
    const int wg = warp >> 2;
    const int row = (warp & 3) * 32 + lane;      // output feature within the tile == TMEM lane
    const int col0 = wg * kCols;                 // first token column of this thread
    const int n = n0 + row;
    const bool n_ok = n < p.N;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + col0;
    const float kScaleUp = 1.2676506002282294e30f;     // 2^100
    const float bias_f = __uint_as_float(bias);        // bias * 2^-149

    float acc[kCols];
#pragma unroll
    for (int j = 0; j < kCols; ++j) acc[j] = 0.f;

    // pre-set both accumulator buffers to the bias and hand them to the MMA issuer
#pragma unroll
    for (int a = 0; a < 2; ++a) {
#pragma unroll
      for (int c = 0; c < kNumChunks; ++c) {
        if constexpr (kChunk == 32) tmem_st_fill_32x32(lane_addr + a * BLOCK_M + c * kChunk, bias);
        else tmem_st_fill_32x16(lane_addr + a * BLOCK_M + c * kChunk, bias);
      }
    }
    tmem_st_wait();
    tcgen05_fence_before_sync();
    mbar_arrive(bar_acc_empty(0));
    mbar_arrive(bar_acc_empty(1));

    float s_next = (n_ok && g_begin < g_end) ? __half2float(p.w_scale[static_cast<size_t>(g_begin) * p.N + n]) : 0.f;
    float s_sum = 0.f;   // sum of scaled group scales since the last bias flush
    int gc = 0;
#pragma unroll 1
    for (int g = g_begin; g < g_end; ++g, ++gc) {
      const float s2 = s_next * kScaleUp;
      if (g + 1 < g_end && n_ok) s_next = __half2float(p.w_scale[static_cast<size_t>(g + 1) * p.N + n]);
      const int a = gc & 1;
      if (!wait_bounded(bar_acc_full(a), (gc >> 1) & 1, ctx, kStEpilogueAccFull)) break;
      tcgen05_fence_after_sync();
      const uint32_t buf = lane_addr + a * BLOCK_M;
      constexpr int kBufMask = T::kDoubleBuf ? 1 : 0;
      uint32_t v[kBufMask + 1][kChunk];
      if constexpr (T::kDoubleBuf) {
        if constexpr (kChunk == 32) tmem_ld_32x32(buf, v[0]); else tmem_ld_32x16(buf, v[0]);
      }
#pragma unroll
      for (int c = 0; c < kNumChunks; ++c) {
        if constexpr (!T::kDoubleBuf) {
          if constexpr (kChunk == 32) tmem_ld_32x32(buf + c * kChunk, v[0]); else tmem_ld_32x16(buf + c * kChunk, v[0]);
        }
        tmem_ld_wait();
        if constexpr (T::kDoubleBuf) {
          if (c + 1 < kNumChunks) {
            if constexpr (kChunk == 32) tmem_ld_32x32(buf + (c + 1) * kChunk, v[(c + 1) & 1]);
            else tmem_ld_32x16(buf + (c + 1) * kChunk, v[(c + 1) & 1]);
          }
        }
        if constexpr (kChunk == 32) tmem_st_fill_32x32(buf + c * kChunk, bias);
        else tmem_st_fill_32x16(buf + c * kChunk, bias);
        if (c == kNumChunks - 1) {   // buffer fully read and re-set: hand it back to the MMA issuer
          tmem_st_wait();
          tcgen05_fence_before_sync();
          mbar_arrive(bar_acc_empty(a));
        }
        if constexpr (DUMP) {
          if (n_ok) {
#pragma unroll
            for (int j = 0; j < kChunk; ++j) {
              const int m = m0 + col0 + c * kChunk + j;
              if (m < p.M)
                p.partials[(static_cast<size_t>(g) * p.M + m) * p.N + n] =
                    static_cast<int32_t>(v[c & kBufMask][j]) - static_cast<int32_t>(bias);
            }
          }
        }
#pragma unroll
        for (int j = 0; j < kChunk; ++j)
          acc[c * kChunk + j] = fmaf(s2, __uint_as_float(v[c & kBufMask][j]), acc[c * kChunk + j]);
      }
      s_sum += s2;
      if ((gc % kBiasFlushGroups) == kBiasFlushGroups - 1) {
        const float corr = s_sum * bias_f;
#pragma unroll
        for (int j = 0; j < kCols; ++j) acc[j] -= corr;
        s_sum = 0.f;
      }
    }
    {
      const float corr = s_sum * bias_f;
#pragma unroll
      for (int j = 0; j < kCols; ++j) acc[j] -= corr;
    }

    // ---------------------------------------------------------------- output
    if constexpr (!DUMP) {
      const float kScaleDown = 5.62949953421312e14f;   // 2^49: acc holds (sum_g s P) * 2^-49
      // The operand ring is dead once the last group has been read (all MMAs and all TMA loads are complete):
      // reuse it to transpose the tile.  All epilogue threads must be past their last TMEM read first.
      float* xs_s = reinterpret_cast<float*>(smem + T::kOffXs);
      for (int j = threadIdx.x; j < BLOCK_M; j += T::kEpiThreads)
        xs_s[j] = (m0 + j < p.M) ? __ldg(p.x_scale + m0 + j) * kScaleDown : 0.f;
      named_barrier_sync(1, T::kEpiThreads);
      if (num_splits == 1) {
        uint16_t* st = reinterpret_cast<uint16_t*>(smem);   // [BLOCK_M][128] in the output dtype
#pragma unroll
        for (int j = 0; j < kCols; ++j) {
          if ((j & 15) == 0) asm volatile("" ::: "memory");   // keep the scale loads from being hoisted en bloc
          const float y = acc[j] * xs_s[col0 + j];
          st[(col0 + j) * kTileN + row] = p.out_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(y))
                                                     : __half_as_ushort(__float2half_rn(y));
        }
        named_barrier_sync(1, T::kEpiThreads);
        uint16_t* outp = reinterpret_cast<uint16_t*>(p.out);
        const bool vec_ok = (n0 + kTileN <= p.N) && (p.ld_out % 8 == 0) &&
                            ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
        if (vec_ok) {
          // 16 threads x 16 bytes cover one 256-byte row of the tile
          for (int idx = threadIdx.x; idx < BLOCK_M * 16; idx += T::kEpiThreads) {
            const int j = idx >> 4, ch = idx & 15;
            const int m = m0 + j;
            if (m < p.M)
              *reinterpret_cast<uint4*>(outp + static_cast<size_t>(m) * p.ld_out + n0 + ch * 8) =
                  *reinterpret_cast<const uint4*>(st + j * kTileN + ch * 8);
          }
        } else {
          for (int idx = threadIdx.x; idx < BLOCK_M * kTileN; idx += T::kEpiThreads) {
            const int j = idx >> 7, r = idx & 127;
            const int m = m0 + j;
            if (m < p.M && n0 + r < p.N) outp[static_cast<size_t>(m) * p.ld_out + n0 + r] = st[j * kTileN + r];
          }
        }
      } else {
        float* red = reinterpret_cast<float*>(smem);        // [BLOCK_M][128] fp32
#pragma unroll
        for (int j = 0; j < kCols; ++j) red[(col0 + j) * kTileN + row] = acc[j];
      }
    }
  }

  if constexpr (!DUMP) {
    if (num_splits > 1) {
      // split-K: fixed-order reduction over the cluster through distributed shared memory
      const float kScaleDown = 5.62949953421312e14f;
      __syncwarp();
      cluster_sync_all();
      if (warp < EPI_WGS * 4) {
        const float* red = reinterpret_cast<const float*>(smem);
        const uint32_t my_rank = cluster_ctarank();
        const int row = threadIdx.x & 127;
        const int wg = warp >> 2;
        const int n = n0 + row;
        uint16_t* outp = reinterpret_cast<uint16_t*>(p.out);
        // token rows are dealt round-robin to (cluster rank, epilogue warpgroup)
        for (int j = static_cast<int>(my_rank) * EPI_WGS + wg; j < BLOCK_M; j += num_splits * EPI_WGS) {
          const int m = m0 + j;
          if (m >= p.M) break;
          const uint32_t local = smem_u32(red + j * kTileN + row);
          float sum = 0.f;
          for (int r = 0; r < num_splits; ++r) sum += ld_dsmem_f32(map_to_cta(local, r));
          const float y = sum * (__ldg(p.x_scale + m) * kScaleDown);
          if (n < p.N)
            outp[static_cast<size_t>(m) * p.ld_out + n] = p.out_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(y))
                                                                     : __half_as_ushort(__float2half_rn(y));
        }
      }
      __syncwarp();
      cluster_sync_all();   // peers may still be reading this CTA's shared memory until here
    }
  }

  // ---------------------------------------------------------------- teardown
  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) {
    tcgen05_fence_after_sync();
    tmem_dealloc(tmem_base, T::kTmemCols);
  }
}

}  // namespace sk
