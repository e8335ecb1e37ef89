// The W2A8 GEMM kernel for sm_100a.
//
// One CTA computes a tile of 128 output features x BLOCK_M tokens over a range of scale groups:
//   1. a producer warp brings, per 128-wide K block, one 4 KiB block of tiled 2-bit weights (bulk TMA copy)
//      and one BLOCK_M x 128 int8 activation tile (tensor-map TMA, 128-byte swizzle) into a ring of shared
//      memory stages guarded by mbarriers;
//   2. expander warps turn the 2-bit codes into int8 bytes (code - zero_point) with a byte-permute look-up
//      (prmt), written straight into the 128-byte-swizzled K-major layout the tensor core reads;
//   3. two MMA warps, taking the scale groups in turn, issue tcgen05.mma kind::i8 (128 x BLOCK_M x 32 per
//      instruction): the weights are the "A"/M operand, the tokens the "B"/N operand, int32 accumulators live in
//      tensor memory, one accumulator buffer per scale group (ACC_BUFS buffers, so later groups accumulate while
//      earlier ones drain);
//   4. one or two epilogue warpgroups read each finished group from tensor memory (lane = output feature,
//      column = token), multiply by that feature's group scale (a per-thread scalar) and accumulate in fp32;
//      at the end the per-token activation scale is applied, the tile is transposed through shared memory
//      and leaves through one TMA store per destination (16-byte coalesced stores by the threads where the
//      output's alignment rules that out).
//
// Integer -> float without a conversion instruction, and without ever resetting an accumulator:
//   * every accumulator buffer is pre-set ONCE per tile to the bias B = 2^22 and the MMAs always accumulate, so
//     after group g buffer b = g mod ACC_BUFS holds the running sum  D_g = B + sum_{g' <= g, g' = g mod ACC_BUFS} P_g'
//     with 0 < D < 2^23 (the host refuses K ranges whose running sums could leave that interval);
//   * read as an IEEE float those bits are the denormal D * 2^-149, exactly;
//   * summation by parts turns  sum_g s_g P_g  into  sum_g (s_g - s_{g+ACC_BUFS}) (D_g - B)  (s = 0 past the
//     end), so the epilogue needs ONE fused multiply-add per value, acc += ((s_g - s_{g+ACC_BUFS}) * 2^100) *
//     asfloat(D_g); the B term is the same for every token of a thread and is removed once per 16 groups.
// Re-setting a buffer per group instead (tcgen05.st) costs more tensor-memory write bandwidth than the whole
// epilogue has to spare.  The debug entry point stores the running sums; the host differences them into P.
//
// The producer and MMA warps run their loops warp-uniformly (all lanes wait, one elected lane issues) and keep
// the loop bodies short: a single warp retires dependent instructions several cycles apart.  Even so one issuing
// thread needs longer for its commits, barrier polls and loop between two groups than the tensor core needs for a
// group, hence the two issuers.  mbarriers count one arrival per warp.
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
constexpr int kWpBytes = kTileN * kBlockK / 4;   // 4096: tiled 2-bit block
constexpr int kWxBytes = kTileN * kBlockK;       // 16384: expanded int8 block
constexpr long long kWaitLimitCycles = 1000000000ll;  // default: every mbarrier wait gives up after 1e9 SM cycles (0.5-0.8 s)
constexpr int kScalePrefetchGroups = 8;   // group scales are pulled into L2 this many groups before they are loaded
constexpr int kBiasFlushGroups = 16;  // the bias term is subtracted from the accumulators this often

// device status codes: role * 16 + barrier kind
enum : int {
  kStProducerEmpty = 0x11,
  kStExpanderFull = 0x21, kStExpanderEmpty = 0x22,
  kStMmaLdFull = 0x31, kStMmaExFull = 0x32, kStMmaAccEmpty = 0x33,
  kStEpilogueAccFull = 0x41, kStEpilogueScales = 0x42,
  kStDrain = 0x51,
  kStStreamSlots = 0x61   // balanced-split decode kernel: host and device disagree on how a tile is cut (never expected)
};

// Optional in-kernel timeline (compiled only with -DSK_TRACE): CTA (0,0,0) stores SM clock stamps.
#ifdef SK_TRACE
#ifndef SK_TRACE_CTA
#define SK_TRACE_CTA 0
#endif
#define SK_TRACE_EVENT(role, idx)                                                                 \
  do {                                                                                            \
    if (p.trace && blockIdx.x == SK_TRACE_CTA && blockIdx.y == 0 && blockIdx.z == 0 && (idx) < 64) \
      p.trace[(role) * 64 + (idx)] = clock64();                                                   \
  } while (0)
#define SK_TRACE_BASE (((tile - tile_first) / tile_step) * (kb_end - kb_begin))   /* events of earlier tiles */
#else
#define SK_TRACE_EVENT(role, idx) do { } while (0)
#define SK_TRACE_BASE 0
#endif

// Tensor maps of the further destinations of an output tile (peer GPUs' buffers): [M][N] 16-bit, box 128 x BLOCK_M.
struct ExtraOutMaps { CUtensorMap map[7]; };

struct GemmParams {
  const uint8_t* w_tiled;     // [n_tiles][k_blocks][4096]
  const __half* w_scale;      // [groups, N]
  const __half* w_scale_tiled;  // [n_tiles][k_blocks][128] copy of w_scale (group size 128; rows past N zero), or nullptr
  const float* x_scale;       // [M]
  void* out;                  // [M, ld_out] half or bf16
  void* out_extra[7];         // further destinations of the same tile (peer GPUs' buffers), same ld_out
  int n_extra;                // how many of them are used
  int scatter_rows;           // > 0: row scatter -- token rows [d * scatter_rows, (d + 1) * scatter_rows) go to destination d
                              // ONLY (0 = out, d = out_extra[d - 1]), at rows scatter_row0 + (m - d * scatter_rows) there
  int scatter_row0;
  int32_t* partials;          // [groups, M, N] (debug mode) or nullptr
  int* status;                // device status word
  long long ld_out;
  int M, N, K;
  int k_blocks;               // ceil(K / 128)
  int steps_per_group;        // G / 32
  int groups;                 // K / G
  int zero_point;
  int out_bf16;
  int tma_out;                // 1: the output tile leaves through TMA stores (tensor maps of every destination given)
  int n_tiles;                // ceil(N / 128)
  int num_tiles;              // n_tiles * token tiles
  long long wait_limit;       // SM cycles after which a wait inside the kernel gives up (kWaitLimitCycles by default)
  int fault_skip_kb;          // failure-path test hook: the producer leaves out the copies of this K block of its
                              // range (-1: off), so that the waits for them run into the limit
  int mix_tiles1;             // decode kernel with clusters, mixed launch: tiles that get a CTA of their own (multiple of 4)
  int mix_split;              // ... and how the further tiles are split (4 or 2); 0: plain launch
  // balanced-split decode kernel (w2a8_stream.cuh): partial sums of tiles shared between CTAs
  float* stream_scratch;      // [n_tiles][stream_slots][token tile][128] fp32
  int* stream_counters;       // [n_tiles][4]: contributions received per (tile, epilogue warp); zero between launches
  int stream_slots;           // slots per tile = the most CTAs that can share one tile
#ifdef SK_TRACE
  long long* trace;           // [8][64] clock stamps of CTA (0,0,0)
#endif
};

template <int BLOCK_M, int EPI_WGS, int EXP_WARPS, int LSTAGES, int ESTAGES, int ACC_BUFS, bool A_TMEM = false,
          bool PERSIST = false>
struct KernelTraits {
  static constexpr int kEpiWarps = EPI_WGS * 4;
  static constexpr int kWarps = ((kEpiWarps + EXP_WARPS + 2 + 3) / 4) * 4;   // whole warpgroups
  static constexpr int kThreads = kWarps * 32;
  static constexpr int kEpiThreads = EPI_WGS * 128;
  static constexpr int kExpThreads = EXP_WARPS * 32;
  static constexpr int kRowsPerExpThread = EXP_WARPS == 2 ? 2 : 1;   // with 8 warps a thread expands half a row
  static constexpr int kColsPerWg = BLOCK_M / EPI_WGS;           // accumulators per epilogue thread
  static constexpr int kChunk = kColsPerWg >= 32 ? 32 : 16;      // TMEM columns per tcgen05.ld
  static constexpr int kNumChunks = kColsPerWg / kChunk;
  // A_TMEM: the expanded weights go to tensor memory (32 columns per stage) instead of shared memory, which takes
  // 32 KB of shared-memory traffic per K block off the pipe the tensor core reads its other operand through.
  static constexpr int kAccCols = ACC_BUFS * BLOCK_M;
  static constexpr int kATmemCol0 = kAccCols;                       // first column of the A stages
  static constexpr int kTmemNeed = kAccCols + (A_TMEM ? ESTAGES * 32 : 0);
  static constexpr uint32_t kTmemCols = kTmemNeed <= 32 ? 32 : kTmemNeed <= 64 ? 64 : kTmemNeed <= 128 ? 128
                                        : kTmemNeed <= 256 ? 256 : 512;
  static constexpr int kXBytes = BLOCK_M * kBlockK;
  static constexpr int kOffX = 0;
  static constexpr int kOffWx = kOffX + LSTAGES * kXBytes;
  static constexpr int kOffWp = kOffWx + (A_TMEM ? 0 : ESTAGES * kWxBytes);
  // Persistent CTAs write the output through a staging area of their own (the ring belongs to the next tile by
  // then): kStageTokens tokens x 128 features x 16 bit per epilogue warpgroup, sent with TMA stores.
  static constexpr int kStageTokens = 64;
  static constexpr int kStageBytes = kStageTokens * kTileN * 2;                  // 16 KB per warpgroup
  static constexpr int kOffStage = kOffWp + LSTAGES * kWpBytes;
  static constexpr int kOffBar = kOffStage + (PERSIST ? EPI_WGS * kStageBytes : 0);
  static constexpr int kNumBars = 2 * LSTAGES + 2 * ESTAGES + 2 * ACC_BUFS;
  static constexpr int kOffMisc = kOffBar + kNumBars * 8;
  static constexpr int kOffXs = kOffMisc + 16;                   // fp32 [2][BLOCK_M]: x_scale of the tile's tokens
  static constexpr int kTotal = kOffXs + 2 * BLOCK_M * 4;
  static constexpr int kDynamicBytes = kTotal + 1024;            // slack for 1024-byte alignment of the base
  // After the main loop the operand ring is dead and is reused for the output tile
  // (fp32 [BLOCK_M][128] for the split-K reduction, 16-bit [BLOCK_M][128] otherwise).
  static_assert(BLOCK_M * kTileN * 4 <= kOffStage, "output staging must fit in the operand ring");
  static_assert(!PERSIST || (EPI_WGS == 2 && (BLOCK_M / EPI_WGS) % kStageTokens == 0), "persistent output rounds");
  static_assert(kColsPerWg % kChunk == 0 && kNumChunks >= 1, "bad epilogue split");
  static_assert(EXP_WARPS == 2 || EXP_WARPS == 4 || EXP_WARPS == 8, "expander warps");
  static_assert((ACC_BUFS & (ACC_BUFS - 1)) == 0 && kTmemNeed <= 512, "TMEM");
  static_assert(!A_TMEM || EXP_WARPS == 4, "TMEM-resident weights: one expander warp per lane quadrant");
  // The expanded-weight ring is indexed like the load ring (stage i of one is stage i of the other): when the TMA
  // data of stage i has landed, the MMAs that read the previous contents of stage i -- operands AND expanded
  // weights -- have completed, because the producer refills a stage only after their commit.  That saves the
  // expanders one barrier wait and one arrival per K block.
  // With fewer expanded stages than load stages (a deep load ring hides the TMA latency; expanded stages cost
  // 16 KB of shared memory or 32 TMEM columns each) a separate "expanded stage free" barrier is needed.
  static constexpr bool kTied = (ESTAGES == LSTAGES);
  static_assert(ESTAGES <= LSTAGES, "expanded stages");
  // Register budgets.  With two epilogue warpgroups the epilogue threads hold kColsPerWg accumulators plus two
  // sets of TMEM-load registers and take registers from the other warpgroup(s) with setmaxnreg.  The CTA's pool
  // is what it was given at launch (kLaunchRegs per thread); setmaxnreg.inc BLOCKS until the pool can serve it,
  // so the budgets must add up to no more than the pool or the kernel hangs:
  //   BLOCK_M 256, 4 expander warps: 512 threads, 128 at launch -> epilogue 224, expanders 32, control 32
  //   BLOCK_M 256, 2 expander warps: 384 threads, 168 at launch -> epilogue 224, expanders + control 56
  //   BLOCK_M 128:                   512 threads, 128 at launch -> epilogue 168, others 88
  static constexpr bool kUseSetMaxNReg = (EPI_WGS == 2);
  static constexpr int kLaunchRegs = (65536 / kThreads) / 8 * 8;
  static constexpr bool kBig = kColsPerWg > 96;
  static constexpr int kEpiRegs = kBig ? 224 : 168;
  static constexpr int kExpRegs = kBig ? 32 : 88;                         // warpgroup holding the expander warps
  static constexpr int kCtlRegs = kBig ? (kThreads == 384 ? 56 : 32) : 88;   // warpgroup holding producer + MMA warps
  static constexpr int kExpWgThreads = (EXP_WARPS == 4) ? 128 : 0;        // expanders have a warpgroup of their own
  static_assert(!kUseSetMaxNReg ||
                    kEpiThreads * kEpiRegs + kExpWgThreads * kExpRegs +
                            (kThreads - kEpiThreads - kExpWgThreads) * kCtlRegs <= kThreads * kLaunchRegs,
                "setmaxnreg budgets exceed the registers the CTA owns");
  // Load chunk c+1 from TMEM while chunk c is consumed (two sets of load registers; worth 1-3 % on the 256-token
  // tile, where it needs the epilogue's 224-register budget).
  static constexpr bool kDoubleBuf = (kNumChunks > 1);
  static constexpr int kMinBlocks = (BLOCK_M <= 32) ? 2 : 1;
  static_assert(kMinBlocks * kThreads <= 2048, "threads per SM");
  static_assert(kEpiWarps + EXP_WARPS + 3 <= kWarps, "room for the producer warp and two MMA-issuing warps");
};

struct WaitCtx {
  volatile int* abort_flag;  // shared memory
  int* status;               // global
  long long limit;           // SM cycles
};

// Slow path of a bounded wait (inlined: a real call inside a kernel that re-partitions registers with setmaxnreg
// does not compile); the fast path in wait_bounded is a single poll.
// The limit is counted on the SM clock (%globaltimer costs about a microsecond per read).
__device__ __forceinline__ bool wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code,
                                          long long limit) {
  const long long t0 = clock64();
  for (uint32_t spins = 1;; ++spins) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spins & 63u) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > limit) {
        *abort_flag = 1;
        atomicCAS(status, 0, code);
        return false;
      }
    }
  }
}
// Bounded wait.  Returns false if the limit expired here or in any other thread of the CTA.
__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity, const WaitCtx& ctx, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  return wait_slow(bar, parity, ctx.abort_flag, ctx.status, code, ctx.limit);
}

// Bounded wait for a role that is not on the critical path of a K block: sleeps between polls, so that it does not
// take issue slots and integer-pipe cycles from the warps that expand (the expansion saturates the integer pipe).
__device__ __forceinline__ bool wait_bounded_relaxed(uint32_t bar, uint32_t parity, const WaitCtx& ctx, int code,
                                                     unsigned sleep_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    __nanosleep(sleep_ns);
    if (mbar_try_wait(bar, parity)) return true;
    if (*ctx.abort_flag) return false;
    if (clock64() - t0 > ctx.limit) {
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

// Output staging: COUNT tokens of one feature (this thread's accumulators acc[j0 .. j0+COUNT), times the token scales
// xs[0 .. COUNT) in shared memory) -> 16-bit values at dst[t * kTileN], t = 0 .. COUNT-1.
// Two tokens per conversion instruction (the f32 -> f16 conversion unit runs at a quarter of the FMA rate), the
// scales fetched four at a time, eight tokens in flight so that the load/multiply/convert/store latencies overlap.
template <int COUNT, bool BF16, int NACC>
__device__ __forceinline__ void stage_tokens(const float (&acc)[NACC], int j0, const float* xs, uint16_t* dst) {
  static_assert(COUNT % 8 == 0, "tokens per staging call");
#pragma unroll
  for (int b = 0; b < COUNT; b += 8) {
    const float4 s0 = *reinterpret_cast<const float4*>(xs + b);
    const float4 s1 = *reinterpret_cast<const float4*>(xs + b + 4);
    const float y[8] = {acc[j0 + b] * s0.x,     acc[j0 + b + 1] * s0.y, acc[j0 + b + 2] * s0.z, acc[j0 + b + 3] * s0.w,
                        acc[j0 + b + 4] * s1.x, acc[j0 + b + 5] * s1.y, acc[j0 + b + 6] * s1.z, acc[j0 + b + 7] * s1.w};
    uint32_t h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if constexpr (BF16) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(y[2 * i], y[2 * i + 1]);
        h[i] = *reinterpret_cast<const uint32_t*>(&v);
      } else {
        const __half2 v = __floats2half2_rn(y[2 * i], y[2 * i + 1]);
        h[i] = *reinterpret_cast<const uint32_t*>(&v);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      dst[(b + 2 * i) * kTileN] = static_cast<uint16_t>(h[i]);
      dst[(b + 2 * i + 1) * kTileN] = static_cast<uint16_t>(h[i] >> 16);
    }
  }
}

// Tile order.  CTAs are handed out in the order of their linear tile number, so tiles that run at the same time
// should share operands in L2: tiles are numbered in bands of kBandTiles token tiles, feature tile by feature tile
// inside a band.  The ~148 tiles in flight then read few feature tiles' weights (each reused by the whole band)
// and kBandTiles token tiles' activations, instead of streaming the whole weight matrix once per token tile.
constexpr int kBandTiles = 4;
struct TileCoord { int n_tile, m_tile; };
__device__ __forceinline__ TileCoord tile_coord(int tile, int n_tiles, int num_tiles) {
  const int m_tiles = num_tiles / n_tiles;
  const int per_band = kBandTiles * n_tiles;
  const int band = tile / per_band;
  const int r = tile - band * per_band;
  const int h = min(kBandTiles, m_tiles - band * kBandTiles);   // token tiles in this band (the last may be short)
  TileCoord c;
  c.n_tile = r / h;
  c.m_tile = band * kBandTiles + (r - c.n_tile * h);
  return c;
}

template <int CHUNK>
__device__ __forceinline__ void tmem_ld_chunk(uint32_t taddr, uint32_t (&v)[CHUNK]) {
  if constexpr (CHUNK == 32) tmem_ld_32x32(taddr, v); else tmem_ld_32x16(taddr, v);
}
template <int CHUNK>
__device__ __forceinline__ void tmem_fill_chunk(uint32_t taddr, uint32_t value) {
  if constexpr (CHUNK == 32) tmem_st_fill_32x32(taddr, value); else tmem_st_fill_32x16(taddr, value);
}

template <int BLOCK_M, int EPI_WGS, int EXP_WARPS, int LSTAGES, int ESTAGES, int ACC_BUFS, bool DUMP, bool A_TMEM = false,
          bool PERSIST = false>
__global__ void __launch_bounds__(KernelTraits<BLOCK_M, EPI_WGS, EXP_WARPS, LSTAGES, ESTAGES, ACC_BUFS, A_TMEM, PERSIST>::kThreads,
                                  KernelTraits<BLOCK_M, EPI_WGS, EXP_WARPS, LSTAGES, ESTAGES, ACC_BUFS, A_TMEM, PERSIST>::kMinBlocks)
w2a8_umma_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_out,
                 const __grid_constant__ ExtraOutMaps tmap_extra, const GemmParams p) {
  using T = KernelTraits<BLOCK_M, EPI_WGS, EXP_WARPS, LSTAGES, ESTAGES, ACC_BUFS, A_TMEM, PERSIST>;
  constexpr int kChunk = T::kChunk;
  constexpr int kNumChunks = T::kNumChunks;
  constexpr int kCols = T::kColsPerWg;
  constexpr uint32_t kStageTxBytes = kWpBytes + T::kXBytes;
  constexpr int kExpWarp0 = T::kEpiWarps;       // first expander warp
  constexpr int kProducerWarp = kExpWarp0 + EXP_WARPS;
  constexpr int kMmaWarp = kProducerWarp + 1;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + T::kOffBar;
  // barrier addresses: consecutive 8-byte slots
  const uint32_t bar_ld_full = bar_base;
  const uint32_t bar_ld_empty = bar_ld_full + 8u * LSTAGES;
  const uint32_t bar_ex_full = bar_ld_empty + 8u * LSTAGES;
  const uint32_t bar_ex_empty = bar_ex_full + 8u * ESTAGES;      // used only when the rings are not tied
  const uint32_t bar_acc_full = bar_ex_empty + 8u * ESTAGES;
  const uint32_t bar_acc_empty = bar_acc_full + 8u * ACC_BUFS;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + T::kOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + T::kOffMisc + 4);
  const WaitCtx ctx{abort_flag, p.status, p.wait_limit};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int split = blockIdx.z;
  const int num_splits = gridDim.z;
  // Tiles are numbered feature-tile fastest.  A persistent CTA walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...:
  // its rings, barrier phases and accumulator buffers simply carry on from one tile to the next, so the loads,
  // the expansion and the MMAs of the next tile start while the epilogue still writes the previous one.
  const int tile_first = static_cast<int>(blockIdx.x + blockIdx.y * gridDim.x);   // persistent: gridDim.y == 1
  const int tile_end = PERSIST ? p.num_tiles : tile_first + 1;
  const int tile_step = PERSIST ? static_cast<int>(gridDim.x) : 1;

  // K range of this CTA, in whole scale groups.
  const int groups_per_split = (p.groups + num_splits - 1) / num_splits;
  const int g_begin = min(split * groups_per_split, p.groups);
  const int g_end = min(g_begin + groups_per_split, p.groups);
  const int ks_begin = g_begin * p.steps_per_group;
  const int ks_end = g_end * p.steps_per_group;
  const int kb_begin = ks_begin / 4;
  const int kb_end = (ks_end + 3) / 4;

  // running sums stay inside (-2^22, 2^22): checked on the host (kMaxKPerAccBuf)
  const uint32_t bias = 1u << 22;

  // ---------------------------------------------------------------- set-up
  if (threadIdx.x == 0) SK_TRACE_EVENT(4, 0);
  // Every mbarrier counts ONE arrival per participating warp (lane 0, after __syncwarp): arrivals on one
  // barrier are serialised shared-memory atomics.
  if (threadIdx.x == 0) {
    for (int i = 0; i < LSTAGES; ++i) {
      mbar_init(bar_ld_full + 8 * i, 1);           // TMA transaction bytes
      mbar_init(bar_ld_empty + 8 * i, 1);          // tcgen05.commit of the MMAs that read the stage
    }
    for (int i = 0; i < ESTAGES; ++i) {
      mbar_init(bar_ex_full + 8 * i, EXP_WARPS);   // expanded weights of the stage are in place
      mbar_init(bar_ex_empty + 8 * i, 1);          // commit of the MMAs that read them (untied rings only)
    }
    for (int i = 0; i < ACC_BUFS; ++i) { mbar_init(bar_acc_full + 8 * i, 1); mbar_init(bar_acc_empty + 8 * i, T::kEpiWarps); }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == kProducerWarp && lane == 0) {
    prefetch_tensormap(&tmap_x);
    if constexpr (PERSIST) prefetch_tensormap(&tmap_out);
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), T::kTmemCols);
    tmem_relinquish();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) SK_TRACE_EVENT(4, 1);

  if (warp >= kExpWarp0) {
    if constexpr (T::kUseSetMaxNReg) {
      if (EXP_WARPS == 4 && warp < kProducerWarp) setmaxnreg_dec<T::kExpRegs>();
      else setmaxnreg_dec<T::kCtlRegs>();
    }
    if (warp == kProducerWarp) {
      // ============================================================ producer (whole warp loops, one lane issues)
      uint32_t dst_wp = smem_base + T::kOffWp, dst_x = smem_base + T::kOffX;
      uint32_t full = bar_ld_full, empty = bar_ld_empty;
      int stage = 0, issued = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = tile_first; tile < tile_end && ok; tile += tile_step) {
        const TileCoord tc = tile_coord(tile, p.n_tiles, p.num_tiles);
        const int n_tile = tc.n_tile;
        const int m0 = tc.m_tile * BLOCK_M;
        const uint8_t* wsrc = p.w_tiled + (static_cast<size_t>(n_tile) * p.k_blocks + kb_begin) * kWpBytes;
        for (int kcoord = kb_begin * kBlockK; kcoord < kb_end * kBlockK; kcoord += kBlockK) {
          ok = wait_bounded_relaxed(empty, phase ^ 1, ctx, kStProducerEmpty, 100);   // not urgent: the ring is several K blocks deep
          if (!ok) break;
          if (elect_one() && kcoord != (kb_begin + p.fault_skip_kb) * kBlockK) {
            SK_TRACE_EVENT(0, issued);
            mbar_arrive_expect_tx(full, kStageTxBytes);
            bulk_load_1d(dst_wp, wsrc, kWpBytes, full);
            tma_load_2d(dst_x, &tmap_x, kcoord, m0, full);
          }
          __syncwarp();
          wsrc += kWpBytes; ++issued;
          if (++stage == LSTAGES) {
            stage = 0; phase ^= 1;
            dst_wp = smem_base + T::kOffWp; dst_x = smem_base + T::kOffX; full = bar_ld_full; empty = bar_ld_empty;
          } else {
            dst_wp += kWpBytes; dst_x += T::kXBytes; full += 8; empty += 8;
          }
        }
      }
      if (!ok) {
        // Gave up: wait (bounded) until every copy this warp started has landed, so that none is in
        // flight into this CTA's shared memory when the CTA exits.
        const long long t0 = clock64();
        const int first = issued > LSTAGES ? issued - LSTAGES : 0;
        for (int i = first; i < issued; ++i) {
          const int l = i % LSTAGES;
          const uint32_t ph = (i / LSTAGES) & 1;
          while (!mbar_try_wait(bar_ld_full + 8 * l, ph)) {
            if (clock64() - t0 > ctx.limit) { atomicCAS(p.status, 0, kStDrain); break; }
          }
        }
      }
      __syncwarp();
    } else if (warp == kMmaWarp || warp == kMmaWarp + 1) {
      // ============================================================ MMA issuers (whole warp loops, one lane issues)
      // TWO warps take the scale groups in turn.  Between the MMAs of one group and those of the next a single
      // issuing thread spends ~800 cycles on its commits, loop and barrier polls -- longer than the tensor core
      // needs for what is queued -- so with one issuer the tensor pipe idles about half the time; with two, one
      // warp's overhead overlaps the other's issue.  Consecutive groups use different accumulator buffers and
      // different stages, and tcgen05.commit tracks the issuing thread's own MMAs, so the two streams are independent.
      const int mma_id = warp - kMmaWarp;
      constexpr uint32_t idesc = make_idesc_i8(kTileN, BLOCK_M, /*a_signed=*/true, /*b_signed=*/true);
      const uint64_t a_desc0 = make_kmajor_sw128_desc(smem_base + T::kOffWx);
      const uint64_t b_desc0 = make_kmajor_sw128_desc(smem_base + T::kOffX);
      int l = 0, e = 0, ab = 0;                 // load stage, expanded stage, accumulator buffer
      uint32_t lph = 0, eph = 0, aph = 0;       // their phases
      bool ok = true;
      if (p.steps_per_group == 4) {
        // one K block == one scale group: four MMAs and three commits per iteration, nothing else
        int turn = 0;                             // whose group this is (alternates over all K blocks of all tiles)
        for (int tile = tile_first; tile < tile_end && ok; tile += tile_step)
        for (int kb = kb_begin; kb < kb_end; ++kb, turn ^= 1) {
          if (turn != mma_id) {                   // the other warp's group: only keep the ring state in step
            if (++l == LSTAGES) { l = 0; lph ^= 1; }
            if (++e == ESTAGES) { e = 0; eph ^= 1; }
            if (++ab == ACC_BUFS) { ab = 0; aph ^= 1; }
            continue;
          }
#ifdef SK_TRACE_MMA_FINE
          if (lane == 0 && kb - kb_begin >= 8 && kb - kb_begin < 16) SK_TRACE_EVENT(5, (kb - kb_begin - 8) * 8 + 0);
          ok = wait_bounded(bar_ld_full + 8 * l, lph, ctx, kStMmaLdFull);
          if (lane == 0 && kb - kb_begin >= 8 && kb - kb_begin < 16) SK_TRACE_EVENT(5, (kb - kb_begin - 8) * 8 + 1);
          ok = ok && wait_bounded(bar_ex_full + 8 * e, eph, ctx, kStMmaExFull);
          if (lane == 0 && kb - kb_begin >= 8 && kb - kb_begin < 16) SK_TRACE_EVENT(5, (kb - kb_begin - 8) * 8 + 2);
          ok = ok && wait_bounded(bar_acc_empty + 8 * ab, aph, ctx, kStMmaAccEmpty);
          if (lane == 0 && kb - kb_begin >= 8 && kb - kb_begin < 16) SK_TRACE_EVENT(5, (kb - kb_begin - 8) * 8 + 3);
#else
          ok = wait_bounded(bar_ld_full + 8 * l, lph, ctx, kStMmaLdFull) &&
               wait_bounded(bar_ex_full + 8 * e, eph, ctx, kStMmaExFull) &&
               wait_bounded(bar_acc_empty + 8 * ab, aph, ctx, kStMmaAccEmpty);
#endif
          if (!ok) break;
          tcgen05_fence_after_sync();
          if (elect_one()) {
            const uint64_t a_desc = a_desc0 + static_cast<uint64_t>(e * (kWxBytes >> 4));
            const uint64_t b_desc = b_desc0 + static_cast<uint64_t>(l * (T::kXBytes >> 4));
            const uint32_t d = tmem_base + ab * BLOCK_M;
            // +2 in the (address >> 4) field advances 32 bytes along K inside the 128-byte swizzle row
            if constexpr (A_TMEM) {
              const uint32_t a_t = tmem_base + T::kATmemCol0 + e * 32;   // 8 columns per 32-wide K step
              umma_i8_ts(d, a_t, b_desc, idesc, 1u);
              umma_i8_ts(d, a_t + 8, b_desc + 2, idesc, 1u);
              umma_i8_ts(d, a_t + 16, b_desc + 4, idesc, 1u);
              umma_i8_ts(d, a_t + 24, b_desc + 6, idesc, 1u);
            } else {
              umma_i8(d, a_desc, b_desc, idesc, 1u);
              umma_i8(d, a_desc + 2, b_desc + 2, idesc, 1u);
              umma_i8(d, a_desc + 4, b_desc + 4, idesc, 1u);
              umma_i8(d, a_desc + 6, b_desc + 6, idesc, 1u);
            }
#ifdef SK_TRACE_MMA_FINE
            if (kb - kb_begin >= 8 && kb - kb_begin < 16) SK_TRACE_EVENT(5, (kb - kb_begin - 8) * 8 + 4);
#endif
            umma_commit(bar_acc_full + 8 * ab);
            umma_commit(bar_ld_empty + 8 * l);
            if constexpr (!T::kTied) umma_commit(bar_ex_empty + 8 * e);
#ifdef SK_TRACE_MMA_FINE
            if (kb - kb_begin >= 8 && kb - kb_begin < 16) SK_TRACE_EVENT(5, (kb - kb_begin - 8) * 8 + 5);
#endif
            SK_TRACE_EVENT(2, SK_TRACE_BASE + kb - kb_begin);
          }
          __syncwarp();
          if (++l == LSTAGES) { l = 0; lph ^= 1; }
          if (++e == ESTAGES) { e = 0; eph ^= 1; }
          if (++ab == ACC_BUFS) { ab = 0; aph ^= 1; }
        }
      } else {
        // general group sizes (32, 64, 256, ...): one issuer, tracking the position inside the group per 32-wide K step
        int pos = 0;
        if (mma_id == 0)
        for (int tile = tile_first; tile < tile_end && ok; tile += tile_step)
        for (int kb = kb_begin; kb < kb_end && ok; ++kb) {
          ok = wait_bounded(bar_ld_full + 8 * l, lph, ctx, kStMmaLdFull) &&
               wait_bounded(bar_ex_full + 8 * e, eph, ctx, kStMmaExFull);
          if (!ok) break;
          tcgen05_fence_after_sync();
          const uint64_t a_desc = a_desc0 + static_cast<uint64_t>(e * (kWxBytes >> 4));
          const uint64_t b_desc = b_desc0 + static_cast<uint64_t>(l * (T::kXBytes >> 4));
#pragma unroll 1
          for (int s = 0; s < 4; ++s) {
            const int ks = kb * 4 + s;
            if (ks < ks_begin || ks >= ks_end) continue;
            if (pos == 0) {
              ok = wait_bounded(bar_acc_empty + 8 * ab, aph, ctx, kStMmaAccEmpty);
              if (!ok) break;
              tcgen05_fence_after_sync();
            }
            const bool last = (pos == p.steps_per_group - 1);
            if (elect_one()) {
              if constexpr (A_TMEM)
                umma_i8_ts(tmem_base + ab * BLOCK_M, tmem_base + T::kATmemCol0 + e * 32 + 8 * s, b_desc + 2 * s, idesc, 1u);
              else
                umma_i8(tmem_base + ab * BLOCK_M, a_desc + 2 * s, b_desc + 2 * s, idesc, 1u);
              if (last) umma_commit(bar_acc_full + 8 * ab);
            }
            __syncwarp();
            if (last) {
              pos = 0;
              if (++ab == ACC_BUFS) { ab = 0; aph ^= 1; }
            } else {
              ++pos;
            }
          }
          if (!ok) break;
          if (elect_one()) {
            umma_commit(bar_ld_empty + 8 * l);
            if constexpr (!T::kTied) umma_commit(bar_ex_empty + 8 * e);
          }
          __syncwarp();
          if (++l == LSTAGES) { l = 0; lph ^= 1; }
          if (++e == ESTAGES) { e = 0; eph ^= 1; }
        }
      }
      __syncwarp();
    } else if (warp < kProducerWarp) {
      // ============================================================ expanders (one or two weight rows per thread)
      const int et = threadIdx.x - kExpWarp0 * 32;             // expander thread index
      constexpr bool kHalfRows = (EXP_WARPS == 8);             // 8 warps: a thread expands half a row
      const int row0 = kHalfRows ? (et >> 1) : et * T::kRowsPerExpThread;
      const int half = kHalfRows ? (et & 1) : 0;
      const int zp = p.zero_point;
      const uint32_t lut = (static_cast<uint32_t>(0 - zp) & 0xffu) | ((static_cast<uint32_t>(1 - zp) & 0xffu) << 8) |
                           ((static_cast<uint32_t>(2 - zp) & 0xffu) << 16) | ((static_cast<uint32_t>(3 - zp) & 0xffu) << 24);
      int l = 0, e = 0;
      uint32_t lph = 0, eph = 0;
      // Row r of the expanded tile lives at r * 128; its 16-byte chunk c sits at chunk (c ^ (r & 7)).  The row base
      // is 128-aligned, so  base + ((c ^ sw) << 4) == (base + (sw << 4)) ^ (c << 4): one XOR per store.
      uint32_t wx_off[T::kRowsPerExpThread], wp_off[T::kRowsPerExpThread];
#pragma unroll
      for (int rr = 0; rr < T::kRowsPerExpThread; ++rr) {
        const int row = row0 + rr;
        wx_off[rr] = T::kOffWx + row * 128 + ((row & 7) << 4);
        wp_off[rr] = T::kOffWp + row * 16 + half * 2048;
      }
      bool ok = true;
      for (int tile = tile_first; tile < tile_end && ok; tile += tile_step)
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        // The loads below must not be issued before the wait has been seen to succeed: a load that does not depend
        // on the poll's predicate can be served before the barrier state is sampled and return stale bytes.
        ok = wait_bounded(bar_ld_full + 8 * l, lph, ctx, kStExpanderFull);
        if (!ok) break;
        if constexpr (!T::kTied) {
          ok = wait_bounded(bar_ex_empty + 8 * e, eph ^ 1, ctx, kStExpanderEmpty);
          if (!ok) break;
        }
        const uint32_t wp = smem_base + wp_off[0] + l * kWpBytes;
        const uint4 q0 = ld_shared_v4(wp);
        const uint4 q1 = kHalfRows ? make_uint4(0, 0, 0, 0) : ld_shared_v4(wp + 2048);
        if constexpr (A_TMEM) {
          // this thread's row (= its TMEM lane): 32 bytes of codes in, 128 int8 bytes out as 32 TMEM columns
          const uint32_t words[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
          uint32_t a_row[32];
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint4 o = expand16(words[c], lut);
            a_row[4 * c] = o.x; a_row[4 * c + 1] = o.y; a_row[4 * c + 2] = o.z; a_row[4 * c + 3] = o.w;
          }
          tmem_st_32x32(tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + T::kATmemCol0 + e * 32, a_row);
          tmem_st_wait();
          tcgen05_fence_before_sync();
        } else {
          const uint32_t wx = smem_base + wx_off[0] + e * kWxBytes;
          if constexpr (kHalfRows) {
            // 16 bytes in (codes 64 half .. +63 of this row), 64 bytes out
            const uint32_t words[4] = {q0.x, q0.y, q0.z, q0.w};
#pragma unroll
            for (int c = 0; c < 4; ++c) st_shared_v4(wx ^ ((4 * half + c) << 4), expand16(words[c], lut));
          } else {
            // 2 x 16 bytes in (codes 0..63 and 64..127 of this row), 128 bytes out
            const uint32_t words[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
            for (int c = 0; c < 8; ++c) st_shared_v4(wx ^ (c << 4), expand16(words[c], lut));
          }
          if constexpr (T::kRowsPerExpThread == 2) {    // two rows per thread: the second row, read after the wait
            const uint8_t* wp2 = smem + wp_off[1] + l * kWpBytes;
            const uint32_t wx2 = smem_base + wx_off[1] + e * kWxBytes;
            const uint4 r0 = *reinterpret_cast<const uint4*>(wp2);
            const uint4 r1 = *reinterpret_cast<const uint4*>(wp2 + 2048);
            const uint32_t words2[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
            for (int c = 0; c < 8; ++c) st_shared_v4(wx2 ^ (c << 4), expand16(words2[c], lut));
          }
          fence_proxy_async_smem();   // generic-proxy stores -> visible to the tensor core's async proxy
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_ex_full + 8 * e);
        if (threadIdx.x == kExpWarp0 * 32) SK_TRACE_EVENT(1, SK_TRACE_BASE + kb - kb_begin);
        if (++l == LSTAGES) { l = 0; lph ^= 1; }
        if (++e == ESTAGES) { e = 0; eph ^= 1; }
      }
    }
  } else {
    // ============================================================ epilogue
    // warp w: TMEM lanes 32 (w % 4) .. +31 (hardware rule), token columns of warpgroup w / 4
    if constexpr (T::kUseSetMaxNReg) setmaxnreg_inc<T::kEpiRegs>();
    const int wg = warp >> 2;
    const int row = (warp & 3) * 32 + lane;      // output feature within the tile == TMEM lane
    const int col0 = wg * kCols;                 // first token column of this thread
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + col0;
    const float kScaleUp = 1.2676506002282294e30f;     // 2^100
    const float bias_f = __uint_as_float(bias);        // bias * 2^-149

    // pre-set every accumulator buffer to the bias and hand them to the MMA issuer
#pragma unroll
    for (int a = 0; a < ACC_BUFS; ++a) {
#pragma unroll
      for (int c = 0; c < kNumChunks; ++c) tmem_fill_chunk<kChunk>(lane_addr + a * BLOCK_M + c * kChunk, bias);
    }
    tmem_st_wait();
    tcgen05_fence_before_sync();
    __syncwarp();
    if (lane == 0) {
#pragma unroll
      for (int a = 0; a < ACC_BUFS; ++a) mbar_arrive(bar_acc_empty + 8 * a);
    }
    int ab = 0, tile_parity = 0;
    uint32_t aph = 0;
    bool epi_ok = true;

    for (int tile = tile_first; tile < tile_end && epi_ok; tile += tile_step) {
    const TileCoord tc = tile_coord(tile, p.n_tiles, p.num_tiles);
    const int n0 = tc.n_tile * kTileN;
    const int m0 = tc.m_tile * BLOCK_M;
    const int n = n0 + row;
    const bool n_ok = n < p.N;
    const bool more_tiles = PERSIST && tile + tile_step < tile_end;   // the buffers must be pre-set again for the next tile

    float acc[kCols];
#pragma unroll
    for (int j = 0; j < kCols; ++j) acc[j] = 0.f;
    float* xs_tile = reinterpret_cast<float*>(smem + T::kOffXs) + (tile_parity ? BLOCK_M : 0);
    if constexpr (PERSIST) {
      // x_scale * 2^49 of this tile's tokens; read after the named barrier that precedes the output.  The buffer
      // of the tile before last is free: every epilogue thread passed that tile's barrier before it got here.
      for (int j = threadIdx.x; j < BLOCK_M; j += T::kEpiThreads)
        xs_tile[j] = (m0 + j < p.M) ? __ldg(p.x_scale + m0 + j) * 5.62949953421312e14f : 0.f;
      tile_parity ^= 1;
    }

    // group scales s_g .. s_{g+ACC_BUFS} in a register ring, loaded one group ahead of their first use (0 past the
    // end).  The ring keeps the raw fp16 bits: converting at load time would stall on the global load right away.
    // A load that misses L2 would still stall the loop one group later (the ring is shifted by register moves), so
    // every row is pulled into L2 kScalePrefetchGroups groups earlier with a prefetch, which occupies no register.
    const unsigned short* sp =
        reinterpret_cast<const unsigned short*>(p.w_scale) + static_cast<size_t>(g_begin) * p.N + (n_ok ? n : 0);
    int g_load = g_begin;                       // next group whose scale is fetched
    auto load_scale = [&]() -> unsigned short {
      const unsigned short r = (n_ok && g_load < g_end) ? __ldg(sp) : static_cast<unsigned short>(0);
#ifndef SK_NO_SCALE_PREFETCH
      if (g_load + kScalePrefetchGroups < g_end)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(sp + static_cast<size_t>(kScalePrefetchGroups) * p.N));
#endif
      sp += p.N; ++g_load;
      return r;
    };
    for (int i = ACC_BUFS + 1; i < kScalePrefetchGroups && g_begin + i < g_end; ++i)
      asm volatile("prefetch.global.L2 [%0];" ::"l"(sp + static_cast<size_t>(i) * p.N));
    unsigned short sr[ACC_BUFS + 1];
#pragma unroll
    for (int i = 0; i <= ACC_BUFS; ++i) sr[i] = load_scale();
    float s_sum = 0.f;   // sum of the coefficients since the last bias flush
    int flush = 0;
    // TMEM loads are software-pipelined across the chunks of a group: while chunk c is consumed the load of chunk
    // c + 1 is in flight (prefetching across groups as well costs more registers than the epilogue has).
    // (the debug variant keeps one set of load registers: it also holds the dump addresses)
    constexpr bool kDB = T::kDoubleBuf && !DUMP;
    constexpr int kBufMask = kDB ? 1 : 0;
    uint32_t v[kBufMask + 1][kChunk];
#pragma unroll 1
    for (int g = g_begin; g < g_end && epi_ok; ++g) {
      // coefficient of this group's running sum
      const float s2 = (__half2float(__ushort_as_half(sr[0])) - __half2float(__ushort_as_half(sr[ACC_BUFS]))) * kScaleUp;
#pragma unroll
      for (int i = 0; i < ACC_BUFS; ++i) sr[i] = sr[i + 1];
      sr[ACC_BUFS] = load_scale();
      const uint32_t buf = lane_addr + ab * BLOCK_M;
      // the last groups of a tile keep their buffers until these are back at the bias for the next tile (below)
      const bool keep_buf = more_tiles && g >= g_end - ACC_BUFS;
      if (threadIdx.x == 0) SK_TRACE_EVENT(7, (g - g_begin) * 8 + 0);
      epi_ok = wait_bounded(bar_acc_full + 8 * ab, aph, ctx, kStEpilogueAccFull);
      if (!epi_ok) break;
      if (threadIdx.x == 0) SK_TRACE_EVENT(7, (g - g_begin) * 8 + 1);
      tcgen05_fence_after_sync();
      if constexpr (kDB) tmem_ld_chunk<kChunk>(buf, v[0]);
      int ab_next = ab + 1;
      uint32_t aph_next = aph;
      if (ab_next == ACC_BUFS) { ab_next = 0; aph_next ^= 1; }
#pragma unroll
      for (int c = 0; c < kNumChunks; ++c) {
        if constexpr (!kDB) tmem_ld_chunk<kChunk>(buf + c * kChunk, v[0]);
        tmem_ld_wait();
        if (threadIdx.x == 0 && c < 4) SK_TRACE_EVENT(7, (g - g_begin) * 8 + 2 + c);
        if constexpr (kDB) {
          if (c + 1 < kNumChunks) tmem_ld_chunk<kChunk>(buf + (c + 1) * kChunk, v[(c + 1) & kBufMask]);
        }
        if (c == kNumChunks - 1 && !keep_buf) {   // buffer fully read: hand it back to the MMA issuer (it keeps accumulating)
          tcgen05_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_acc_empty + 8 * ab);
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
      if (threadIdx.x == 0) SK_TRACE_EVENT(3, SK_TRACE_BASE + g - g_begin);
      s_sum += s2;
      if (++flush == kBiasFlushGroups) {
        const float corr = s_sum * bias_f;
#pragma unroll
        for (int j = 0; j < kCols; ++j) acc[j] -= corr;
        s_sum = 0.f; flush = 0;
      }
      ab = ab_next; aph = aph_next;
    }
    if (threadIdx.x == 0 && tile == tile_first) SK_TRACE_EVENT(6, 0);
    if (more_tiles && epi_ok) {
      // back to the bias for the next tile: the buffers of the last ACC_BUFS groups (all of them, if the tile had
      // fewer groups: the untouched ones are at the bias already), then hand them to the MMA issuer
      const int used = (g_end - g_begin) < ACC_BUFS ? (g_end - g_begin) : ACC_BUFS;
      int b = ab;
      for (int i = 0; i < used; ++i) {
        b = (b == 0) ? ACC_BUFS - 1 : b - 1;
#pragma unroll
        for (int cc = 0; cc < kNumChunks; ++cc) tmem_fill_chunk<kChunk>(lane_addr + b * BLOCK_M + cc * kChunk, bias);
      }
      tmem_st_wait();
      tcgen05_fence_before_sync();
      __syncwarp();
      b = ab;
      for (int i = 0; i < used; ++i) {
        b = (b == 0) ? ACC_BUFS - 1 : b - 1;
        if (lane == 0) mbar_arrive(bar_acc_empty + 8 * b);
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
      if constexpr (PERSIST) {
        // Straight from the registers: a warp writes 32 consecutive features (64 bytes) of one token per store.
        // The shared-memory ring is busy with the next tile, whose MMAs run while these stores are issued.
        // The token scales were staged in shared memory at the start of the tile (two buffers, by tile parity).
        // Each warpgroup sends its tokens in rounds of kStageTokens through its own staging buffer: convert and
        // transpose into [token][feature], then one thread issues a TMA store (which clips at the edges of the
        // output) and the warpgroup goes on; the buffer is reused once that store has read it.
        if (threadIdx.x == 0 && tile == tile_first) SK_TRACE_EVENT(6, 1);
        named_barrier_sync(1, T::kEpiThreads);
        if (threadIdx.x == 0 && tile == tile_first) SK_TRACE_EVENT(6, 2);
        const float* xs = xs_tile + col0;
        const uint32_t stage_addr = smem_base + T::kOffStage + wg * T::kStageBytes;
        uint16_t* stage = reinterpret_cast<uint16_t*>(smem + T::kOffStage + wg * T::kStageBytes);
        const bool leader = (threadIdx.x & 127) == 0;
#pragma unroll
        for (int r = 0; r < kCols / T::kStageTokens; ++r) {
          if (leader) bulk_wait_group_read0();
          named_barrier_sync(2 + wg, 128);
          if (threadIdx.x == 0 && tile == tile_first) SK_TRACE_EVENT(6, 3 + 4 * r);
          if (p.out_bf16) stage_tokens<T::kStageTokens, true>(acc, r * T::kStageTokens, xs + r * T::kStageTokens, stage + row);
          else stage_tokens<T::kStageTokens, false>(acc, r * T::kStageTokens, xs + r * T::kStageTokens, stage + row);
          if (threadIdx.x == 0 && tile == tile_first) SK_TRACE_EVENT(6, 4 + 4 * r);
          fence_proxy_async_smem();
          named_barrier_sync(2 + wg, 128);
          if (threadIdx.x == 0 && tile == tile_first) SK_TRACE_EVENT(6, 5 + 4 * r);
          if (leader) {
            tma_store_2d(&tmap_out, n0, m0 + col0 + r * T::kStageTokens, stage_addr);
            bulk_commit_group();
          }
          if (threadIdx.x == 0 && tile == tile_first) SK_TRACE_EVENT(6, 6 + 4 * r);
          // further destinations (peer GPUs): plain 16-byte stores out of the staging buffer
          for (int d = 0; d < p.n_extra; ++d) {
            uint16_t* outp = reinterpret_cast<uint16_t*>(p.out_extra[d]);
            for (int idx = threadIdx.x & 127; idx < T::kStageTokens * 16; idx += 128) {
              const int jj = idx >> 4, ch = idx & 15;
              const int m = m0 + col0 + r * T::kStageTokens + jj;
              if (m < p.M)
                *reinterpret_cast<uint4*>(outp + static_cast<size_t>(m) * p.ld_out + n0 + ch * 8) =
                    *reinterpret_cast<const uint4*>(stage + jj * kTileN + ch * 8);
            }
          }
        }
        continue;
      }
      // The operand ring is dead once the last group has been read (all MMAs and all TMA loads are complete):
      // reuse it to transpose the tile.  All epilogue threads must be past their last TMEM read first.
      float* xs_s = reinterpret_cast<float*>(smem + T::kOffXs);
      for (int j = threadIdx.x; j < BLOCK_M; j += T::kEpiThreads)
        xs_s[j] = (m0 + j < p.M) ? __ldg(p.x_scale + m0 + j) * kScaleDown : 0.f;
      named_barrier_sync(1, T::kEpiThreads);
      if (threadIdx.x == 0) SK_TRACE_EVENT(4, 2);
      if (num_splits == 1) {
        uint16_t* st = reinterpret_cast<uint16_t*>(smem);   // [BLOCK_M][128] in the output dtype
        if (p.out_bf16) stage_tokens<kCols, true>(acc, 0, xs_s + col0, st + col0 * kTileN + row);
        else stage_tokens<kCols, false>(acc, 0, xs_s + col0, st + col0 * kTileN + row);
        if (p.tma_out) fence_proxy_async_smem();   // the staged tile is read by the TMA (async proxy)
        named_barrier_sync(1, T::kEpiThreads);
        // destination 0 is this GPU's buffer; the others are peer-mapped buffers of the other ranks (stores over
        // NVLink, so the all-gather of the output overlaps the GEMM tile by tile)
        // With row scatter the tile has ONE destination, chosen by its token rows, and lands at another row there.
        int d_first = 0, d_last = p.n_extra, m_dst = m0;
        if (p.scatter_rows > 0) {
          d_first = d_last = m0 / p.scatter_rows;
          m_dst = p.scatter_row0 + (m0 - d_first * p.scatter_rows);
        }
        if (p.tma_out) {
          // one TMA store per destination moves the whole staged tile (clipped at the edges of the output) while
          // the CTA winds down; the thread only waits until the stores have READ shared memory
          if (threadIdx.x == 0) {
            for (int d = d_first; d <= d_last; ++d) tma_store_2d(d == 0 ? &tmap_out : &tmap_extra.map[d - 1], n0, m_dst, smem_base);
            bulk_commit_group();
            bulk_wait_group_read0();
          }
        } else
        for (int d = d_first; d <= d_last; ++d) {
          uint16_t* outp = reinterpret_cast<uint16_t*>(d == 0 ? p.out : p.out_extra[d - 1]);
          const bool vec_ok = (n0 + kTileN <= p.N) && (p.ld_out % 8 == 0) &&
                              ((reinterpret_cast<uintptr_t>(outp) & 15) == 0);
          if (vec_ok) {
            // 16 threads x 16 bytes cover one 256-byte row of the tile
            for (int idx = threadIdx.x; idx < BLOCK_M * 16; idx += T::kEpiThreads) {
              const int j = idx >> 4, ch = idx & 15;
              if (m0 + j < p.M)
                *reinterpret_cast<uint4*>(outp + static_cast<size_t>(m_dst + j) * p.ld_out + n0 + ch * 8) =
                    *reinterpret_cast<const uint4*>(st + j * kTileN + ch * 8);
            }
          } else {
            for (int idx = threadIdx.x; idx < BLOCK_M * kTileN; idx += T::kEpiThreads) {
              const int j = idx >> 7, r = idx & 127;
              if (m0 + j < p.M && n0 + r < p.N) outp[static_cast<size_t>(m_dst + j) * p.ld_out + n0 + r] = st[j * kTileN + r];
            }
          }
        }
      } else {
        float* red = reinterpret_cast<float*>(smem);        // [BLOCK_M][128] fp32
#pragma unroll
        for (int j = 0; j < kCols; ++j) red[(col0 + j) * kTileN + row] = acc[j];
      }
    }
    }   // tiles
    if constexpr (PERSIST) {
      if ((threadIdx.x & 127) == 0) bulk_wait_group0();   // this thread's TMA stores are complete
    }
  }

  if constexpr (!DUMP) {
    if (num_splits > 1) {
      // split-K: fixed-order reduction over the cluster through distributed shared memory
      const float kScaleDown = 5.62949953421312e14f;
      __syncwarp();
      cluster_sync_all();
      if (warp < T::kEpiWarps) {
        const float* red = reinterpret_cast<const float*>(smem);
        const uint32_t my_rank = cluster_ctarank();
        const int row = threadIdx.x & 127;
        const int wg = warp >> 2;
        const TileCoord tc = tile_coord(tile_first, p.n_tiles, p.num_tiles);   // split-K CTAs own exactly one tile
        const int n0 = tc.n_tile * kTileN;
        const int m0 = tc.m_tile * BLOCK_M;
        const int n = n0 + row;
        uint16_t* outp = reinterpret_cast<uint16_t*>(p.out);
        // token rows are dealt round-robin to (cluster rank, epilogue warpgroup); every remote load of a row
        // is issued before the first is consumed, and the sum runs in rank order (deterministic)
        for (int j = static_cast<int>(my_rank) * EPI_WGS + wg; j < BLOCK_M; j += num_splits * EPI_WGS) {
          const int m = m0 + j;
          if (m >= p.M) break;
          const uint32_t local = smem_u32(red + j * kTileN + row);
          float part[8];
#pragma unroll
          for (int r = 0; r < 8; ++r) part[r] = (r < num_splits) ? ld_dsmem_f32(map_to_cta(local, r)) : 0.f;
          float sum = 0.f;
#pragma unroll
          for (int r = 0; r < 8; ++r) sum += part[r];
          const float y = sum * (__ldg(p.x_scale + m) * kScaleDown);
          if (n < p.N) {
            const uint16_t bits = p.out_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(y))
                                             : __half_as_ushort(__float2half_rn(y));
            outp[static_cast<size_t>(m) * p.ld_out + n] = bits;
            for (int d = 0; d < p.n_extra; ++d)
              reinterpret_cast<uint16_t*>(p.out_extra[d])[static_cast<size_t>(m) * p.ld_out + n] = bits;
          }
        }
      }
      __syncwarp();
      cluster_sync_all();   // peers may still be reading this CTA's shared memory until here
    }
  }

  // ---------------------------------------------------------------- teardown
  tcgen05_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0) SK_TRACE_EVENT(4, 3);
  if (warp == kMmaWarp) {
    tcgen05_fence_after_sync();
    tmem_dealloc(tmem_base, T::kTmemCols);
  }
}

}  // namespace sk
