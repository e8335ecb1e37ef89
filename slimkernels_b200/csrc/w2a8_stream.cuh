// The W2A8 GEMM kernel for decode-sized token counts (M <= 32, one token tile) with a BALANCED split of the K range:
// the default decode kernel on sm_100a, group size 128, even number of K blocks.
//
// w2a8_decode.cuh gives every CTA one feature tile (or 1/2, 1/4, 1/8 of its K range, reduced over a cluster).  Tile
// counts are rarely a multiple of the SM count -- 96 tiles split in two are 192 CTAs on 148 SMs, so 44 SMs carry
// two CTAs and the rest one, and the kernel runs as long as the SMs with double load -- and clusters of 8 (or of a
// size that is not a power of two) cost more than a microsecond of launch time.  Here the whole problem is ONE
// linear sequence of half stages (two 128-wide K blocks of one feature tile; tile-major, which is exactly the order
// of the tiled weight layout in memory), cut into gridDim.x equal ranges, two CTAs per SM.  A range may begin and
// end in the middle of a tile:
//   * a CTA's weights are still one contiguous byte range -- the producer does not know about tiles except for
//     the K coordinate of the activation boxes;
//   * the epilogue handles its range tile by tile ("segments").  At the end of a segment it pre-sets the
//     accumulator set it just read to the bias again before handing it back to the MMA issuers, so the running
//     sums of the next tile start afresh;
//   * a segment that covers a whole tile is written out directly.  Otherwise the warp writes its fp32 partial sums
//     (32 features x TOK tokens) into its slot of a scratch buffer in global memory (L2-resident) and bumps the
//     counter of (tile, warp); the warp that finds the counter complete -- whichever CTA it belongs to -- adds the
//     slots in slot order, so the result does not depend on which CTA came last, scales and stores the outputs,
//     and zeroes the counter for the next launch.  Nobody waits for anybody: no cluster, no spin, no requirement
//     that the CTAs be resident together.
// Everything else (four K blocks per load stage, weights expanded into tensor memory, one commit per half stage,
// two accumulator sets, programmatic dependent launch, bias 2^22 arithmetic) is w2a8_decode.cuh's.
//
// Like the other GEMM kernels this replaces the reference's gemm_device
// (slimkernels/cute/gemm/wgmma_sm90_W2A8.cu:165-424); it shares no code with it.
#pragma once
#include "w2a8_umma.cuh"

namespace sk {

template <int TOK, int EXP_WARPS = 4>
struct StreamTraits {
  static_assert(TOK == 16 || TOK == 32, "token tile of the decode kernels");
  static_assert(EXP_WARPS == 4 || EXP_WARPS == 8 || EXP_WARPS == 16, "expander warps: whole groups of four");
  static constexpr int kCtasPerSm = EXP_WARPS == 4 ? 2 : 1;
  static constexpr int kKbPerStage = 4;                      // K blocks per load stage
  static constexpr int kStages = kCtasPerSm == 2 ? (TOK == 16 ? 4 : 3) : (TOK == 16 ? 8 : 6);
  static constexpr int kGroupsPerSet = 2;                    // scale groups (= K blocks) per accumulator set: a half stage
  static constexpr uint32_t kTmemCols = kCtasPerSm == 2 ? 256 : 512;
  // Accumulator sets.  An MMA of half stage u + kAccSets waits until the epilogue has read half stage u, and from
  // the commit of a half stage to the epilogue's hand-back of its set are 1500-2000 cycles (commit, barrier, two
  // tensor-memory loads), so two sets pace a CTA at ~1100 cycles per half stage whatever the other roles do.
  static constexpr int kAccSets = static_cast<int>(kTmemCols) / 2 / (kGroupsPerSet * TOK);   // half the columns: 4, 8 (16 tokens), 2, 4 (32)
  static constexpr int kAccBufs = kAccSets * kGroupsPerSet;  // accumulator buffers
  static constexpr int kAccCols = kAccBufs * TOK;            // tensor memory: [0, kAccCols) accumulators, then weights
  static constexpr int kACol0 = kAccCols;
  static constexpr int kASubs = (static_cast<int>(kTmemCols) - kAccCols) / 64;   // half-stage buffers of expanded weights
  static constexpr int kXKbBytes = TOK * kBlockK;            // one activation box
  static constexpr int kStageWBytes = kKbPerStage * kWpBytes;
  static constexpr int kStageBytes = kStageWBytes + kKbPerStage * kXKbBytes;
  static constexpr int kOffBar = kStages * kStageBytes;
  static constexpr int kSubRing = 2 * kStages;               // ring of "MMAs of a half stage are complete" barriers
  static constexpr int kNumBars = kStages + kSubRing + kASubs + kAccSets;
  static constexpr int kOffMisc = kOffBar + kNumBars * 8;
  static constexpr int kTotal = kOffMisc + 16;
  static constexpr int kDynamicBytes = kTotal + 1024;        // slack for 1024-byte alignment of the base
  static constexpr int kEpiWarps = 4, kExpWarps = EXP_WARPS;
  static constexpr int kExpGroups = EXP_WARPS / 4;           // a group of four warps (one per 32 tensor-memory lanes) expands a half stage
  static constexpr int kThreads = (kEpiWarps + kExpWarps + 4) * 32;   // + producer + 2 MMA warps + 1 idle
  static constexpr int kSlotFloats = TOK * kTileN;           // one CTA's partial sums of one tile
  static_assert(kCtasPerSm * kDynamicBytes <= 227 * 1024, "shared memory per SM");
};

// The cut of the problem into CTA ranges, shared by host and device: with U half stages in all and G CTAs, CTA c
// owns the half stages [U c / G, U (c + 1) / G).
__host__ __device__ inline long long stream_range_begin(long long units, int ctas, int c) {
  return units * c / ctas;
}
// The CTA that owns half stage x.
__host__ __device__ inline int stream_owner(long long units, int ctas, long long x) {
  return static_cast<int>(((x + 1) * ctas + units - 1) / units) - 1;
}

template <int TOK, int EXP_WARPS>
__global__ void __launch_bounds__((StreamTraits<TOK, EXP_WARPS>::kThreads), (StreamTraits<TOK, EXP_WARPS>::kCtasPerSm))
w2a8_stream_kernel(const __grid_constant__ CUtensorMap tmap_x, const GemmParams p) {
  using T = StreamTraits<TOK, EXP_WARPS>;
  constexpr int S = T::kStages;
  constexpr int GS = T::kGroupsPerSet;
  constexpr int kExpWarp0 = T::kEpiWarps;
  constexpr int kProducerWarp = kExpWarp0 + T::kExpWarps;
  constexpr int kMmaWarp = kProducerWarp + 1;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_ld_full = smem_base + T::kOffBar;            // [S] the copies of a stage have landed
  const uint32_t bar_sub_done = bar_ld_full + 8u * S;             // [2 S] the MMAs of a half stage have completed
  const uint32_t bar_ex_full = bar_sub_done + 8u * T::kSubRing;   // [kASubs] expanded weights of a half stage are in tensor memory
  const uint32_t bar_acc_empty = bar_ex_full + 8u * T::kASubs;    // [2] the epilogue has read (and maybe re-set) the accumulator set
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + T::kOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + T::kOffMisc + 4);
  const WaitCtx ctx{abort_flag, p.status, p.wait_limit};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // this CTA's range: half stages [ub, ue) of the tile-major sequence; K blocks are counted from its beginning
  const int units_per_tile = p.k_blocks >> 1;
  const long long units = static_cast<long long>(p.n_tiles) * units_per_tile;
  const int ctas = static_cast<int>(gridDim.x);
  const long long ub = stream_range_begin(units, ctas, static_cast<int>(blockIdx.x));
  const long long ue = stream_range_begin(units, ctas, static_cast<int>(blockIdx.x) + 1);
  const int num_subs = static_cast<int>(ue - ub);
  const int nkb = 2 * num_subs;
  const int tile0 = static_cast<int>(ub / units_per_tile);
  const int unit_off0 = static_cast<int>(ub - static_cast<long long>(tile0) * units_per_tile);   // half stages into the first tile
  const uint32_t bias = 1u << 22;

  // ---------------------------------------------------------------- set-up
  if (threadIdx.x == 0) SK_TRACE_EVENT(4, 0);
  // Programmatic dependent launch: weights and group scales are constants, so the copies of the first stages'
  // weights go out at once, before tensor memory is allocated and before the CTA's first barrier; every thread that
  // reads activations or token scales or writes outputs or scratch waits for the previous kernel first.
  grid_dep_launch_dependents();
  if (warp == kProducerWarp && lane == 0) {
    for (int i = 0; i < S; ++i) mbar_init(bar_ld_full + 8 * i, 1);
    fence_mbar_init();
    const uint8_t* w = p.w_tiled + static_cast<size_t>(2 * ub) * kWpBytes;
    for (int i = 0, st = 0; i < nkb && st < S; i += T::kKbPerStage, ++st) {
      const int n = min(T::kKbPerStage, nkb - i);
      if (i != p.fault_skip_kb) {   // (failure-path test hook: this stage is never filled)
        const uint32_t full = bar_ld_full + 8 * st;
        mbar_arrive_expect_tx(full, static_cast<uint32_t>(n) * (kWpBytes + T::kXKbBytes));
        bulk_load_1d(smem_base + st * T::kStageBytes, w, static_cast<uint32_t>(n) * kWpBytes, full);
      }
      w += static_cast<size_t>(n) * kWpBytes;
    }
    for (int i = 0; i < T::kSubRing; ++i) mbar_init(bar_sub_done + 8 * i, 1);
    for (int i = 0; i < T::kASubs; ++i) mbar_init(bar_ex_full + 8 * i, 4);
    for (int i = 0; i < T::kAccSets; ++i) mbar_init(bar_acc_empty + 8 * i, T::kEpiWarps);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&tmap_x);
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

  if (warp == kProducerWarp) {
    // ============================================================ producer (whole warp loops, one lane issues)
    const uint8_t* wsrc = p.w_tiled + static_cast<size_t>(2 * ub) * kWpBytes;
    const int kb_off0 = 2 * unit_off0;    // K block of the range's first K block inside its tile
    auto k_coord = [&](int i) { return ((kb_off0 + i) % p.k_blocks) * kBlockK; };
    int stage = 0, issued = 0;
    bool ok = true;
    grid_dep_wait();
    if (elect_one()) {
      for (int i = 0, st = 0; i < nkb && st < S; i += T::kKbPerStage, ++st) {
        if (i == p.fault_skip_kb) continue;
        const int n = min(T::kKbPerStage, nkb - i);
        for (int j = 0; j < n; ++j)
          tma_load_2d(smem_base + st * T::kStageBytes + T::kStageWBytes + j * T::kXKbBytes, &tmap_x, k_coord(i + j), 0,
                      bar_ld_full + 8 * st);
      }
    }
    __syncwarp();
    for (int i = 0; i < nkb && issued < S; i += T::kKbPerStage) {
      wsrc += static_cast<size_t>(min(T::kKbPerStage, nkb - i)) * kWpBytes;
      ++issued;
    }
    // later rounds: a stage is refilled once the MMAs of both its halves (of its previous use) are complete
    for (int i = issued * T::kKbPerStage; i < nkb; i += T::kKbPerStage) {
      const int n = min(T::kKbPerStage, nkb - i);
      {
        const int u = 2 * (issued - S);
        ok = wait_bounded_relaxed(bar_sub_done + 8 * (u % T::kSubRing), (u / T::kSubRing) & 1, ctx, kStProducerEmpty, 200) &&
             wait_bounded_relaxed(bar_sub_done + 8 * ((u + 1) % T::kSubRing), ((u + 1) / T::kSubRing) & 1, ctx, kStProducerEmpty, 200);
        if (!ok) break;
      }
      if (elect_one() && i != p.fault_skip_kb) {
        SK_TRACE_EVENT(0, issued);
        const uint32_t full = bar_ld_full + 8 * stage;
        const uint32_t dst = smem_base + stage * T::kStageBytes;
        mbar_arrive_expect_tx(full, static_cast<uint32_t>(n) * (kWpBytes + T::kXKbBytes));
        bulk_load_1d(dst, wsrc, static_cast<uint32_t>(n) * kWpBytes, full);
        for (int j = 0; j < n; ++j)
          tma_load_2d(dst + T::kStageWBytes + j * T::kXKbBytes, &tmap_x, k_coord(i + j), 0, full);
      }
      __syncwarp();
      wsrc += static_cast<size_t>(n) * kWpBytes;
      ++issued;
      if (++stage == S) stage = 0;
    }
    if (!ok) {
      // Gave up: wait (bounded) until every copy this warp started has landed, so that none is in flight into this
      // CTA's shared memory when the CTA exits.
      const long long t0 = clock64();
      const int first = issued > S ? issued - S : 0;
      for (int i = first; i < issued; ++i) {
        while (!mbar_try_wait(bar_ld_full + 8 * (i % S), (i / S) & 1)) {
          if (clock64() - t0 > ctx.limit) { atomicCAS(p.status, 0, kStDrain); break; }
        }
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp || warp == kMmaWarp + 1) {
    // ============================================================ MMA issuers: two warps take the half stages in turn
    constexpr uint32_t idesc = make_idesc_i8(kTileN, TOK, /*a_signed=*/true, /*b_signed=*/true);
    const uint64_t b_desc0 = make_kmajor_sw128_desc(smem_base + T::kStageWBytes);
    const int mma_id = warp - kMmaWarp;
    bool ok = true;
    grid_dep_wait();   // the MMAs read activations: sit here (no issue slots) rather than poll next to the running kernel
    for (int u = mma_id; u < num_subs; u += 2) {   // one half stage: two K blocks, eight MMAs, one accumulator set
      const int i0 = 2 * u;
      const int q = u >> 1;                     // load stage counter
      const int stage = q % S;
      const int a = u % T::kASubs;              // tensor-memory buffer of expanded weights
      ok = wait_bounded(bar_ld_full + 8 * stage, (q / S) & 1, ctx, kStMmaLdFull) &&
           wait_bounded(bar_ex_full + 8 * a, (u / T::kASubs) & 1, ctx, kStMmaExFull) &&
           wait_bounded(bar_acc_empty + 8 * (u % T::kAccSets), (u / T::kAccSets) & 1, ctx, kStMmaAccEmpty);
      if (!ok) break;
      tcgen05_fence_after_sync();
      if (elect_one()) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int i = i0 + j;
          const uint32_t d = tmem_base + (i % T::kAccBufs) * TOK;
          const uint32_t a_t = tmem_base + T::kACol0 + a * 64 + j * 32;   // 8 columns per 32-wide K step
          const uint64_t b_desc = b_desc0 + static_cast<uint64_t>((stage * T::kStageBytes + (i & 3) * T::kXKbBytes) >> 4);
          // +2 in the (address >> 4) field advances 32 bytes along K inside the 128-byte swizzle row
          umma_i8_ts(d, a_t, b_desc, idesc, 1u);
          umma_i8_ts(d, a_t + 8, b_desc + 2, idesc, 1u);
          umma_i8_ts(d, a_t + 16, b_desc + 4, idesc, 1u);
          umma_i8_ts(d, a_t + 24, b_desc + 6, idesc, 1u);
        }
        umma_commit(bar_sub_done + 8 * (u % T::kSubRing));
        SK_TRACE_EVENT(2, u);
      }
      __syncwarp();
    }
    __syncwarp();
  } else if (warp >= kExpWarp0 && warp < kProducerWarp) {
    // ============================================================ expanders: one weight row (= TMEM lane) per thread
    const int row = (warp & 3) * 32 + lane;
    const int zp = p.zero_point;
    const uint32_t lut = (static_cast<uint32_t>(0 - zp) & 0xffu) | ((static_cast<uint32_t>(1 - zp) & 0xffu) << 8) |
                         ((static_cast<uint32_t>(2 - zp) & 0xffu) << 16) | ((static_cast<uint32_t>(3 - zp) & 0xffu) << 24);
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + T::kACol0;
    const int group = (warp - kExpWarp0) >> 2;     // the groups take the half stages in turn
    bool ok = true;
    grid_dep_wait();   // a stage is complete only with its activations: do not poll next to the running kernel
    for (int u = group; u < num_subs && ok; u += T::kExpGroups) {
      const int q = u >> 1;                    // load stage counter
      const int stage = q % S;
      const int a = u % T::kASubs;
      // The loads below must not be issued before the waits have been seen to succeed: a load that does not depend
      // on the poll's predicate can be served before the barrier state is sampled and return stale bytes.
      ok = wait_bounded(bar_ld_full + 8 * stage, (q / S) & 1, ctx, kStExpanderFull);
      if (ok && u >= T::kASubs) {   // the buffer is free once the MMAs that read its previous contents are complete
        const int v = u - T::kASubs;
        ok = wait_bounded(bar_sub_done + 8 * (v % T::kSubRing), (v / T::kSubRing) & 1, ctx, kStExpanderEmpty);
      }
      if (!ok) break;
      tcgen05_fence_after_sync();
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const uint32_t wp = smem_base + stage * T::kStageBytes + (2 * (u & 1) + j) * kWpBytes + row * 16;
        const uint4 q0 = ld_shared_v4(wp);            // codes 0..63 of this row
        const uint4 q1 = ld_shared_v4(wp + 2048);     // codes 64..127
        const uint32_t words[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        uint32_t a_row[32];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 o = expand16(words[c], lut);
          a_row[4 * c] = o.x; a_row[4 * c + 1] = o.y; a_row[4 * c + 2] = o.z; a_row[4 * c + 3] = o.w;
        }
        tmem_st_32x32(t_row + a * 64 + j * 32, a_row);
      }
      tmem_st_wait();
      tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_ex_full + 8 * a);
      if (threadIdx.x == kExpWarp0 * 32) SK_TRACE_EVENT(1, u);
    }
  } else if (warp < T::kEpiWarps) {
    // ============================================================ epilogue: TMEM lane = output feature
    const int row = warp * 32 + lane;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    const float kScaleUp = 1.2676506002282294e30f;     // 2^100
    const float kScaleDown = 5.62949953421312e14f;     // 2^49
    const float bias_f = __uint_as_float(bias);        // bias * 2^-149

    // pre-set the accumulator columns to the bias and hand both sets to the MMA issuers
#pragma unroll
    for (int c = 0; c < T::kAccCols; c += 32) tmem_st_fill_32x32(lane_addr + c, bias);
    tmem_st_wait();
    tcgen05_fence_before_sync();
    __syncwarp();
    if (lane == 0)
      for (int i = 0; i < T::kAccSets; ++i) mbar_arrive(bar_acc_empty + 8 * i);

    if (warp == 0 && lane < TOK && lane < p.M)   // the token scales are read at the end of a segment: have them in L2 by then
      asm volatile("prefetch.global.L2 [%0];" ::"l"(p.x_scale + lane));

    const unsigned short* w_scale = reinterpret_cast<const unsigned short*>(p.w_scale);
    // this warp's 64-byte segment of the first scale rows of a tile's range, pulled into L2
    auto prefetch_rows = [&](int tile, int kb0, int count) {
      const int seg = min(tile * kTileN + warp * 32, p.N - 1);
      const unsigned short* base = w_scale + static_cast<size_t>(kb0) * p.N + seg;
      for (int g = lane; g < count; g += 32)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(base + static_cast<size_t>(g) * p.N));
    };
    prefetch_rows(tile0, 2 * unit_off0, min(nkb, 3 * GS + T::kAccBufs));

    // The tiles this CTA shares with others can only be its first and its last: which CTAs share them, and this
    // CTA's slot among them (worked out here, while the first copies are in flight).
    const int tile_last = static_cast<int>((ue - 1) / units_per_tile);
    auto first_cta_of = [&](int tile) { return stream_owner(units, ctas, static_cast<long long>(tile) * units_per_tile); };
    auto last_cta_of = [&](int tile) { return stream_owner(units, ctas, static_cast<long long>(tile + 1) * units_per_tile - 1); };
    const int shared_first[2] = {first_cta_of(tile0), first_cta_of(tile_last)};
    const int shared_count[2] = {last_cta_of(tile0) - shared_first[0] + 1, last_cta_of(tile_last) - shared_first[1] + 1};
    int pending_tile[2];      // partial sums written but not yet counted
    int pending_which[2];
    int num_pending = 0;

    // one token tile of one feature row: scaled, converted and stored to every destination
    auto store_row = [&](int n, const float (&val)[TOK]) {
      // all token scales first: the compiler cannot move a load above a store that might alias it, and one
      // dependent global load per stored row would serialise the tail
      float xs[TOK];
#pragma unroll
      for (int t = 0; t < TOK; ++t) xs[t] = (t < p.M) ? __ldg(p.x_scale + t) * kScaleDown : 0.f;
      for (int d = 0; d <= p.n_extra; ++d) {
        uint16_t* outp = reinterpret_cast<uint16_t*>(d == 0 ? p.out : p.out_extra[d - 1]) + n;
#pragma unroll
        for (int t = 0; t < TOK; ++t) {
          if (t < p.M) {
            const float y = val[t] * xs[t];
            *outp = p.out_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(y)) : __half_as_ushort(__float2half_rn(y));
          }
          outp += p.ld_out;
        }
      }
    };

    grid_dep_wait();   // nothing completes before the activations exist: do not poll next to the running kernel
    if (lane < TOK && lane < p.M) asm volatile("prefetch.global.L1 [%0];" ::"l"(p.x_scale + lane));
    bool ok = true;
    int si = 0;                       // half stage (= accumulator set use) of this CTA's range
    int tile = tile0, unit_off = unit_off0;
    while (si < num_subs) {
      // ---------------------------------------------------------- one segment: this CTA's share of one tile
      const int seg_units = min(num_subs - si, units_per_tile - unit_off);
      const int seg_kb = 2 * seg_units;
      const int n = tile * kTileN + row;
      const bool n_ok = n < p.N;
      // group scales: coefficient of group g is (s_g - s_{g + kAccBufs}) * 2^100 (s = 0 past the end of the segment);
      // the coefficients of a set are fetched one set ahead, and the rows behind them pulled into L2 earlier still
      const unsigned short* sp = w_scale + static_cast<size_t>(2 * unit_off) * p.N + (n_ok ? n : 0);
      auto scale_at = [&](int g) -> float {
        return (n_ok && g < seg_kb) ? __half2float(__ushort_as_half(__ldg(sp + static_cast<size_t>(g) * p.N))) : 0.f;
      };
      auto coeffs = [&](int sj, float (&c)[GS]) {
#pragma unroll
        for (int j = 0; j < GS; ++j) c[j] = (scale_at(sj * GS + j) - scale_at(sj * GS + j + T::kAccBufs)) * kScaleUp;
        const int ahead = (sj + 3) * GS + T::kAccBufs;      // first row the set after next will need
#pragma unroll
        for (int j = 0; j < GS; ++j)
          if (ahead + j < seg_kb) asm volatile("prefetch.global.L2 [%0];" ::"l"(sp + static_cast<size_t>(ahead + j) * p.N));
      };
      if (si + seg_units < num_subs)   // the first rows of the next segment
        prefetch_rows(tile + 1, 0, min(2 * (num_subs - si - seg_units), 3 * GS + T::kAccBufs));

      float acc[TOK];
#pragma unroll
      for (int t = 0; t < TOK; ++t) acc[t] = 0.f;
      float c_cur[GS], c_next[GS];
      coeffs(0, c_cur);
      float s_sum = 0.f;
      int flush = 0;
      for (int sj = 0; sj < seg_units; ++sj, ++si) {
        coeffs(sj + 1, c_next);      // zeros past the end
        // set si is complete when the MMAs of half stage si are
        ok = wait_bounded(bar_sub_done + 8 * (si % T::kSubRing), (si / T::kSubRing) & 1, ctx, kStEpilogueAccFull);
        if (!ok) break;
        tcgen05_fence_after_sync();
        // the segment's last use of this set, and the range goes on: the next tile starts from the bias again
        const bool reset = (sj + T::kAccSets >= seg_units) && (si + T::kAccSets < num_subs);
        const uint32_t set_addr = lane_addr + (si % T::kAccSets) * (GS * TOK);
#pragma unroll
        for (int j = 0; j < GS; ++j) {
          uint32_t v[TOK];
          if constexpr (TOK == 16) tmem_ld_32x16(set_addr + j * TOK, v);
          else tmem_ld_32x32(set_addr + j * TOK, v);
          tmem_ld_wait();
          if (j == GS - 1) {
            if (reset) {
#pragma unroll
              for (int c = 0; c < GS * TOK; c += 32) tmem_st_fill_32x32(set_addr + c, bias);
              tmem_st_wait();
            }
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acc_empty + 8 * (si % T::kAccSets));   // the MMAs keep accumulating into the set
          }
#pragma unroll
          for (int t = 0; t < TOK; ++t) acc[t] = fmaf(c_cur[j], __uint_as_float(v[t]), acc[t]);
          s_sum += c_cur[j];
          c_cur[j] = c_next[j];
        }
        if (threadIdx.x == 0) SK_TRACE_EVENT(3, si);
        if (++flush == kBiasFlushGroups / GS) {
          const float corr = s_sum * bias_f;
#pragma unroll
          for (int t = 0; t < TOK; ++t) acc[t] -= corr;
          s_sum = 0.f; flush = 0;
        }
      }
      if (!ok) break;
      {
        const float corr = s_sum * bias_f;
#pragma unroll
        for (int t = 0; t < TOK; ++t) acc[t] -= corr;
      }

      // ---------------------------------------------------------- the segment's result
      [[maybe_unused]] const int trace_seg = (tile - tile0) * 4;
      if (threadIdx.x == 0) SK_TRACE_EVENT(7, trace_seg + 0);
      if (seg_units == units_per_tile) {
        if (n_ok) store_row(n, acc);      // the whole tile: straight from the registers
      } else {
        // Shared tile: this warp's partial sums go into the CTA's slot of the tile.  The stores are not waited for
        // here -- the pipeline goes on with the next segment -- and are counted at the end of the CTA's range.
        const int which = tile == tile0 ? 0 : 1;
        const int slot = static_cast<int>(blockIdx.x) - shared_first[which];
        if (shared_count[which] > p.stream_slots || slot < 0 || slot >= shared_count[which] || num_pending == 2) {
          atomicCAS(p.status, 0, kStStreamSlots);   // (host and device disagree on the cut: never)
          ok = false;
          break;
        }
        float* mine = p.stream_scratch + (static_cast<size_t>(tile) * p.stream_slots + slot) * T::kSlotFloats + row;
#pragma unroll
        for (int t = 0; t < TOK; ++t) __stcg(mine + t * kTileN, acc[t]);
        pending_tile[num_pending] = tile;
        pending_which[num_pending] = which;
        ++num_pending;
      }
      if (threadIdx.x == 0) SK_TRACE_EVENT(7, trace_seg + 1);
      ++tile;
      unit_off = 0;
    }

    if (ok && num_pending > 0) {
      // ---------------------------------------------------------- shared tiles: count this warp's contributions;
      // the warp that completes a (tile, warp) counter -- whichever CTA it belongs to -- adds the slots in slot
      // order, so the sum does not depend on who came last, and writes the tile's outputs
      __threadfence();
      __syncwarp();
      if (threadIdx.x == 0) SK_TRACE_EVENT(7, 60);
      int old0 = 0, old1 = 0;
      if (lane == 0) {
        old0 = atomicAdd(p.stream_counters + pending_tile[0] * T::kEpiWarps + warp, 1);
        if (num_pending == 2) old1 = atomicAdd(p.stream_counters + pending_tile[1] * T::kEpiWarps + warp, 1);
      }
      old0 = __shfl_sync(0xffffffffu, old0, 0);
      old1 = __shfl_sync(0xffffffffu, old1, 0);
      if (threadIdx.x == 0) SK_TRACE_EVENT(7, 61);
      for (int k = 0; k < num_pending; ++k) {
        const int expected = shared_count[pending_which[k]];
        if ((k == 0 ? old0 : old1) != expected - 1) continue;
        __threadfence();
        const int t_tile = pending_tile[k];
        const float* src = p.stream_scratch + static_cast<size_t>(t_tile) * p.stream_slots * T::kSlotFloats + row;
        float sum[TOK];
#pragma unroll
        for (int t = 0; t < TOK; ++t) sum[t] = 0.f;
        int s = 0;
        for (; s + 1 < expected; s += 2) {     // two slots' loads in flight at a time
          float a[TOK], b[TOK];
#pragma unroll
          for (int t = 0; t < TOK; ++t) a[t] = __ldcg(src + static_cast<size_t>(s) * T::kSlotFloats + t * kTileN);
#pragma unroll
          for (int t = 0; t < TOK; ++t) b[t] = __ldcg(src + static_cast<size_t>(s + 1) * T::kSlotFloats + t * kTileN);
#pragma unroll
          for (int t = 0; t < TOK; ++t) sum[t] = (sum[t] + a[t]) + b[t];
        }
        if (s < expected) {
#pragma unroll
          for (int t = 0; t < TOK; ++t) sum[t] += __ldcg(src + static_cast<size_t>(s) * T::kSlotFloats + t * kTileN);
        }
        if (lane == 0) p.stream_counters[t_tile * T::kEpiWarps + warp] = 0;   // ready for the next launch
        const int n = t_tile * kTileN + row;
        if (n < p.N) store_row(n, sum);
        if (threadIdx.x == 0) SK_TRACE_EVENT(7, 62 + k);
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  if (threadIdx.x == 0) SK_TRACE_EVENT(4, 3);
  tcgen05_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0) SK_TRACE_EVENT(4, 4);
  if (warp == kMmaWarp) {
    tcgen05_fence_after_sync();
    tmem_dealloc(tmem_base, T::kTmemCols);
  }
}

}  // namespace sk
