// The W2A8 GEMM kernel for decode-sized token counts (M <= 32) on sm_100a, group size 128.
//
// At these sizes the GEMM is a stream of 2-bit weights out of HBM: every weight byte is used once, the tensor-core
// work is small, and what decides the speed is how many bytes each SM keeps in flight and how little the roles
// of a CTA wait for one another.  Compared with the general kernel (w2a8_umma.cuh) this one
//   * moves FOUR 128-wide K blocks per pipeline stage: one 16 KiB bulk copy of tiled weights (consecutive K blocks
//     of a feature tile are contiguous in the tiled layout) plus four small activation boxes, so a CTA has up to
//     64 KiB of weights in flight and the load barriers are passed once per 512 K instead of once per 128;
//   * expands the 2-bit codes straight into TENSOR MEMORY (tcgen05.st), two K blocks ("half a stage") per
//     hand-over, and feeds the MMA its weight operand from there (tcgen05.mma with the A operand in tensor memory,
//     ~10 cycles per 128x16x32 MMA against ~40 with A in shared memory): the expanded int8 weights -- four times
//     the packed bytes -- never touch shared memory;
//   * issues ONE tcgen05.commit per half stage.  Its barrier tells the producer that a stage may be refilled, the
//     expanders that a tensor-memory weight buffer may be overwritten and the epilogue that an accumulator set is
//     complete (an mbarrier phase can be watched by any number of waiters); a commit stalls the issuing thread for
//     hundreds of cycles, several times the MMAs of a decode-sized tile;
//   * keeps two accumulator sets (one per half stage, two scale groups each): the MMAs of one half stage run while
//     the epilogue drains the other with a single wait;
//   * fits two CTAs on an SM (256 tensor-memory columns, < 113 KiB of shared memory, 384 threads each), which
//     smooths out tile counts that are not a multiple of the SM count;
//   * is launched as a programmatic dependent launch: set-up and the weight copies of the first stages start
//     while the previous kernel in the stream is still finishing; activations, token scales and outputs are
//     touched only after griddepcontrol.wait.
// The arithmetic is the one of the general kernel: accumulators pre-set once to the bias 2^22 and never reset,
// running sums read as denormal floats, summation by parts over the four accumulator buffers.  Split-K runs over a
// thread-block cluster: every CTA pushes its partial sums into the shared memory of the CTA that owns the token
// row (remote stores, which do not stall the way remote loads do), one cluster barrier, then every CTA sums its
// rows in rank order (deterministic, no global scratch).
//
// Like the general kernel this replaces the reference's gemm_device
// (slimkernels/cute/gemm/wgmma_sm90_W2A8.cu:165-424); it shares no code with it.
#pragma once
#include "w2a8_umma.cuh"

namespace sk {

template <int TOK>
struct DecodeTraits {
  static_assert(TOK == 16 || TOK == 32, "token tile of the decode kernel");
  static constexpr int kKbPerStage = 4;                      // K blocks per load stage
  static constexpr int kStages = TOK == 16 ? 4 : 3;
  static constexpr int kGroupsPerSet = 2;                    // scale groups (= K blocks) per accumulator set: a half stage
  // Accumulator sets.  The MMAs of half stage u + kAccSets wait until the epilogue has read half stage u, and from
  // the commit of a half stage to the epilogue's hand-back of its set are 1500-2000 cycles (commit, barrier, two
  // tensor-memory loads): with two sets that round trip paces the CTA, whatever the other roles do.
  static constexpr int kAccSets = TOK == 16 ? 4 : 2;
  static constexpr int kAccBufs = kAccSets * kGroupsPerSet;  // accumulator buffers
  static constexpr int kAccCols = kAccBufs * TOK;            // tensor memory: [0, kAccCols) accumulators, then weights
  static constexpr int kACol0 = kAccCols;
  static constexpr uint32_t kTmemCols = 256;
  static constexpr int kASubs = (256 - kAccCols) / 64;       // half-stage buffers of expanded weights: 2
  static constexpr int kXKbBytes = TOK * kBlockK;            // one activation box
  static constexpr int kStageWBytes = kKbPerStage * kWpBytes;
  static constexpr int kStageBytes = kStageWBytes + kKbPerStage * kXKbBytes;
  // split-K: the partial sums other CTAs of the cluster push into this CTA (fp32 [TOK][128]).  With 16 tokens it
  // has memory of its own, because a peer may push while this CTA is still in its main loop; with 32 tokens that
  // would cost the second CTA per SM, so it overlays the operand ring and the CTAs of the cluster meet at one more
  // barrier before anybody pushes.
  static constexpr bool kRedInRing = (TOK == 32);
  static constexpr int kOffRed = kRedInRing ? 0 : kStages * kStageBytes;
  // The group scales of the CTA's K range (fp16 [K blocks][128 features], one bulk copy out of the plan's tiled copy
  // of the scales): the epilogue reads its coefficients from shared memory.  Loaded from global memory one set
  // ahead they cost it an L2 round trip per set -- about as long as everything else in a half stage.
  // With 16 tokens the region behind the ring is [reduction buffer 8 KiB][4 KiB]: a CTA that shares its tile stages
  // up to 16 K blocks of scales behind the reduction buffer, a CTA with a tile of its own (no reduction) up to 48 from
  // the start of the region.  With 32 tokens (reduction buffer inside the ring) the region is 8 KiB of scales.
  static constexpr int kRegionBytes = kRedInRing ? 32 * kTileN * 2 : TOK * kTileN * 4 + 16 * kTileN * 2;
  static constexpr int kOffBar = kStages * kStageBytes + kRegionBytes;
  __host__ __device__ static constexpr int scale_offset(int num_splits) {
    return kStages * kStageBytes + ((kRedInRing || num_splits == 1) ? 0 : TOK * kTileN * 4);
  }
  __host__ __device__ static constexpr int scale_capacity(int num_splits) {   // in K blocks
    return kRedInRing ? 32 : (num_splits == 1 ? kRegionBytes / (kTileN * 2) : 16);
  }
  static_assert(TOK * kTileN * 4 <= kStages * kStageBytes, "reduction buffer");
  static constexpr int kSubRing = 2 * kStages;               // ring of "MMAs of a half stage are complete" barriers
  static constexpr int kNumBars = kStages + kSubRing + kASubs + kAccSets + 1;
  static constexpr int kOffMisc = kOffBar + kNumBars * 8;
  static constexpr int kTotal = kOffMisc + 16;
  static constexpr int kDynamicBytes = kTotal + 1024;        // slack for 1024-byte alignment of the base
  // (eight expander warps -- two groups taking the half stages in turn -- measure the same at 16 tokens and slower at
  // 32, where the kernel then spills under the 64-register budget of two 512-thread CTAs per SM)
  static constexpr int kEpiWarps = 4, kExpWarps = 4;
  static constexpr int kExpGroups = kExpWarps / 4;           // groups of four warps take the half stages in turn
  static constexpr int kThreads = (kEpiWarps + kExpWarps + 4) * 32;   // + producer + 2 MMA warps + 1 idle
  static_assert(2 * (kDynamicBytes + 1024) <= 228 * 1024, "two CTAs per SM (1 KiB per CTA is reserved by the system)");
};

template <int TOK, bool DUMP>
__global__ void __launch_bounds__(DecodeTraits<TOK>::kThreads, 2)
w2a8_decode_kernel(const __grid_constant__ CUtensorMap tmap_x, const GemmParams p) {
  using T = DecodeTraits<TOK>;
  constexpr int S = T::kStages;
  constexpr int GS = T::kGroupsPerSet;
  constexpr int kExpWarp0 = T::kEpiWarps;
  constexpr int kProducerWarp = kExpWarp0 + T::kExpWarps;
  constexpr int kMmaWarp = kProducerWarp + 1;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_ld_full = smem_base + T::kOffBar;    // [S] the copies of a stage have landed
  // [2 S] the MMAs of a half stage (two K blocks) have completed.  ONE tcgen05.commit per half stage serves every
  // consumer of that fact: the producer (the stage may be refilled after its second half), the expanders (the
  // tensor-memory buffer of expanded weights may be overwritten) and the epilogue (an accumulator set is complete
  // after its last half stage).  A commit costs the issuing thread a few hundred cycles, far more than the MMAs of a
  // decode-sized tile, so they are the currency to save.
  const uint32_t bar_sub_done = bar_ld_full + 8u * S;
  const uint32_t bar_ex_full = bar_sub_done + 8u * T::kSubRing;   // [kASubs] expanded weights of a half stage are in tensor memory
  const uint32_t bar_acc_empty = bar_ex_full + 8u * T::kASubs;    // [kAccSets] the epilogue has read the accumulator set
  const uint32_t bar_scale = bar_acc_empty + 8u * T::kAccSets;    // the group scales of the K range have landed
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + T::kOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + T::kOffMisc + 4);
  const WaitCtx ctx{abort_flag, p.status, p.wait_limit};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // Which tile and which share of its K range.  Plain launch: grid (feature tiles, token tiles, splits), one cluster
  // per tile.  Mixed launch (p.mix_split > 0; one token tile; more tiles than SMs): a 1-D grid in clusters of four --
  // the first p.mix_tiles1 tiles get one CTA each (four unrelated tiles per cluster, no reduction), every further
  // tile is split 4 ways over one cluster or 2 ways over half a cluster, so that the tiles beyond one per SM are
  // dealt out in small pieces instead of doubling the load of a few SMs.
  int n_tile = blockIdx.x, split = blockIdx.z, num_splits = gridDim.z;
  int grp_base = 0;          // cluster rank of split 0 of this tile
  const int m0 = blockIdx.y * TOK;
  if (p.mix_split > 0) {
    const int cluster = blockIdx.x >> 2, rank = blockIdx.x & 3;
    const int c1 = p.mix_tiles1 >> 2;
    if (cluster < c1) { n_tile = blockIdx.x; split = 0; num_splits = 1; }
    else if (p.mix_split == 4) { n_tile = p.mix_tiles1 + (cluster - c1); split = rank; num_splits = 4; }
    else { n_tile = p.mix_tiles1 + 2 * (cluster - c1) + (rank >> 1); split = rank & 1; num_splits = 2; grp_base = rank & 2; }
  }
  const int n0 = n_tile * kTileN;

  // K range of this CTA in K blocks (one scale group each)
  const int per_split = (p.groups + num_splits - 1) / num_splits;
  const int kb_begin = min(split * per_split, p.groups);
  const int nkb = min(kb_begin + per_split, p.groups) - kb_begin;
  const uint32_t bias = 1u << 22;
  const bool scales_staged = p.w_scale_tiled != nullptr && nkb <= T::scale_capacity(num_splits) && nkb > 0;
  const int off_scale = T::scale_offset(num_splits);

  // ---------------------------------------------------------------- set-up
  if (threadIdx.x == 0) SK_TRACE_EVENT(4, 0);
  // Programmatic dependent launch: the next kernel in the stream may be scheduled as soon as every CTA of this one
  // got here, and this kernel may itself have started before the previous one finished.  Weights and group scales
  // are constants, so the copies of the first stages' weights go out at once -- from the thread that initialises the
  // barriers, before tensor memory is allocated and before the CTA's first barrier --; every thread that reads
  // activations or token scales or writes outputs waits for the previous kernel first (grid_dep_wait below).
  grid_dep_launch_dependents();
  if (warp == kProducerWarp && lane == 0) {
    for (int i = 0; i < S; ++i) mbar_init(bar_ld_full + 8 * i, 1);
    mbar_init(bar_scale, 1);
    fence_mbar_init();
    if (scales_staged) {
      mbar_arrive_expect_tx(bar_scale, static_cast<uint32_t>(nkb) * (kTileN * 2));
      bulk_load_1d(smem_base + off_scale, p.w_scale_tiled + (static_cast<size_t>(n_tile) * p.k_blocks + kb_begin) * kTileN,
                   static_cast<uint32_t>(nkb) * (kTileN * 2), bar_scale);
    }
    const uint8_t* w = p.w_tiled + (static_cast<size_t>(n_tile) * p.k_blocks + kb_begin) * kWpBytes;
    for (int i = 0, st = 0; i < nkb && st < S; i += T::kKbPerStage, ++st) {
      const int n = min(T::kKbPerStage, nkb - i);
      if (i != p.fault_skip_kb) {   // (failure-path test hook: this stage is never filled)
        const uint32_t full = bar_ld_full + 8 * st;
        SK_TRACE_EVENT(0, st);
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
    const uint8_t* wsrc = p.w_tiled + (static_cast<size_t>(n_tile) * p.k_blocks + kb_begin) * kWpBytes;
    int stage = 0, issued = 0;
    bool ok = true;
    // first round of stages: the weight copies are under way already (set-up); once the previous kernel in the stream
    // is complete, the activation boxes
    grid_dep_wait();
    if (elect_one()) {
      for (int i = 0, st = 0; i < nkb && st < S; i += T::kKbPerStage, ++st) {
        if (i == p.fault_skip_kb) continue;
        const int n = min(T::kKbPerStage, nkb - i);
        for (int j = 0; j < n; ++j)
          tma_load_2d(smem_base + st * T::kStageBytes + T::kStageWBytes + j * T::kXKbBytes, &tmap_x,
                      (kb_begin + i + j) * kBlockK, m0, bar_ld_full + 8 * st);
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
      {   // both half stages of the stage's previous use (they are committed by different warps, in any order)
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
          tma_load_2d(dst + T::kStageWBytes + j * T::kXKbBytes, &tmap_x, (kb_begin + i + j) * kBlockK, m0, full);
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
    // ============================================================ MMA issuers (whole warp loops, one lane issues)
    // Two warps take the half stages in turn: between two half stages one issuing thread spends several hundred
    // cycles on its commit, barrier polls and loop -- more than the MMAs of a decode-sized half stage take -- and
    // consecutive half stages use different accumulator sets and different weight buffers, so the two streams are
    // independent (tcgen05.commit tracks the issuing thread's own MMAs).
    constexpr uint32_t idesc = make_idesc_i8(kTileN, TOK, /*a_signed=*/true, /*b_signed=*/true);
    const uint64_t b_desc0 = make_kmajor_sw128_desc(smem_base + T::kStageWBytes);
    const int mma_id = warp - kMmaWarp;
    bool ok = true;
    const int num_subs = (nkb + 1) >> 1;
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
        const int n = min(2, nkb - i0);
        for (int j = 0; j < n; ++j) {
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
    const int group = (warp - kExpWarp0) >> 2;
    bool ok = true;
    grid_dep_wait();   // a stage is complete only with its activations: do not poll next to the running kernel
    const int num_subs = (nkb + 1) >> 1;
    for (int u = group; u < num_subs && ok; u += T::kExpGroups) {
      const int i = 2 * u;
      const int q = u >> 1;
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
      const int n = min(2, nkb - i);
      for (int j = 0; j < n; ++j) {
        const uint32_t wp = smem_base + stage * T::kStageBytes + ((i & 3) + j) * kWpBytes + row * 16;
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
    const int n = n0 + row;
    const bool n_ok = n < p.N;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    const float kScaleUp = 1.2676506002282294e30f;     // 2^100
    const float kScaleDown = 5.62949953421312e14f;     // 2^49
    const float bias_f = __uint_as_float(bias);        // bias * 2^-149

    // pre-set the accumulator columns to the bias (once) and hand both sets to the MMA issuer
#pragma unroll
    for (int c = 0; c < T::kAccCols; c += 32) tmem_st_fill_32x32(lane_addr + c, bias);
    tmem_st_wait();
    tcgen05_fence_before_sync();
    __syncwarp();
    if (lane == 0)
      for (int i = 0; i < T::kAccSets; ++i) mbar_arrive(bar_acc_empty + 8 * i);

    // group scales: coefficient of group i is (s_i - s_{i + kAccBufs}) * 2^100 (s = 0 past the end of the range);
    // the coefficients of a set are fetched one set ahead, and the rows behind them pulled into L2 earlier still
    const unsigned short* sp =
        reinterpret_cast<const unsigned short*>(p.w_scale) + static_cast<size_t>(kb_begin) * p.N + (n_ok ? n : 0);
    const uint32_t scale_smem = smem_base + off_scale + row * 2;
    auto scale_at = [&](int g) -> float {
      if (scales_staged) {   // (rows past N are zero in the tiled copy)
        if (g >= nkb) return 0.f;
        unsigned short h;
        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(h) : "r"(scale_smem + g * (kTileN * 2)));
        return __half2float(__ushort_as_half(h));
      }
      return (n_ok && g < nkb) ? __half2float(__ushort_as_half(__ldg(sp + static_cast<size_t>(g) * p.N))) : 0.f;
    };
    auto coeffs = [&](int si, float (&c)[GS]) {
#pragma unroll
      for (int j = 0; j < GS; ++j) c[j] = (scale_at(si * GS + j) - scale_at(si * GS + j + T::kAccBufs)) * kScaleUp;
      const int ahead = (si + 3) * GS + T::kAccBufs;      // first row the set after next will need
#pragma unroll
      for (int j = 0; j < GS; ++j)
        if (!scales_staged && ahead + j < nkb) asm volatile("prefetch.global.L2 [%0];" ::"l"(sp + static_cast<size_t>(ahead + j) * p.N));
    };
    if (!DUMP && warp == 0 && lane < TOK && m0 + lane < p.M)   // the token scales are read at the very end: have them in L2 by then
      asm volatile("prefetch.global.L2 [%0];" ::"l"(p.x_scale + m0 + lane));
    if (!scales_staged) {   // rows the first sets need: pull this warp's 64-byte segment of each into L2 now
      const int seg = min(n0 + warp * 32, p.N - 1);
      const unsigned short* base = reinterpret_cast<const unsigned short*>(p.w_scale) + static_cast<size_t>(kb_begin) * p.N + seg;
      for (int g = lane; g < min(nkb, 3 * GS + T::kAccBufs); g += 32)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(base + static_cast<size_t>(g) * p.N));
    }

    float acc[TOK];
#pragma unroll
    for (int t = 0; t < TOK; ++t) acc[t] = 0.f;
    float c_cur[GS], c_next[GS];
    bool ok = true;
    if (scales_staged) ok = wait_bounded(bar_scale, 0, ctx, kStEpilogueScales);
    coeffs(0, c_cur);
    grid_dep_wait();   // nothing completes before the activations exist: do not poll next to the running kernel
    float s_sum = 0.f;
    int flush = 0;
    const int num_sets = (nkb + GS - 1) / GS;
    for (int si = 0; si < num_sets && ok; ++si) {
      coeffs(si + 1, c_next);      // zeros past the end
      // set si is complete when the MMAs of half stage si are
      ok = wait_bounded(bar_sub_done + 8 * (si % T::kSubRing), (si / T::kSubRing) & 1, ctx, kStEpilogueAccFull);
      if (!ok) break;
      tcgen05_fence_after_sync();
      // a set is read one group (TOK columns) per load
#pragma unroll
      for (int j = 0; j < GS; ++j) {
        uint32_t v[TOK];
        if constexpr (TOK == 16) tmem_ld_32x16(lane_addr + (si % T::kAccSets) * (GS * TOK) + j * TOK, v);
        else tmem_ld_32x32(lane_addr + (si % T::kAccSets) * (GS * TOK) + j * TOK, v);
        tmem_ld_wait();
        if (j == GS - 1) {
          tcgen05_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_acc_empty + 8 * (si % T::kAccSets));   // the MMAs keep accumulating into the set
        }
        if constexpr (DUMP) {
          const int g = si * GS + j;
          if (n_ok && g < nkb) {
#pragma unroll
            for (int t = 0; t < TOK; ++t)
              if (m0 + t < p.M)
                p.partials[(static_cast<size_t>(kb_begin + g) * p.M + m0 + t) * p.N + n] =
                    static_cast<int32_t>(v[t]) - static_cast<int32_t>(bias);
          }
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
    {
      const float corr = s_sum * bias_f;
#pragma unroll
      for (int t = 0; t < TOK; ++t) acc[t] -= corr;
    }

    // ---------------------------------------------------------------- output
    if (threadIdx.x == 0) SK_TRACE_EVENT(4, 2);
    grid_dep_wait();   // token scales and outputs belong to the stream's data flow
    if constexpr (!DUMP) {
      if (num_splits == 1) {
        // straight from the registers: a warp writes 32 consecutive features (64 bytes) of one token per store
        if (n_ok && ok) {
          // all token scales first: the compiler cannot move a load above a store that might alias it, and one
          // dependent global load per stored row would serialise the tail
          float xs[TOK];
#pragma unroll
          for (int t = 0; t < TOK; ++t) xs[t] = (m0 + t < p.M) ? __ldg(p.x_scale + m0 + t) * kScaleDown : 0.f;
          for (int d = 0; d <= p.n_extra; ++d) {
            uint16_t* outp = reinterpret_cast<uint16_t*>(d == 0 ? p.out : p.out_extra[d - 1]) +
                             static_cast<size_t>(m0) * p.ld_out + n;
#pragma unroll
            for (int t = 0; t < TOK; ++t) {
              if (m0 + t < p.M) {
                const float y = acc[t] * xs[t];
                *outp = p.out_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(y)) : __half_as_ushort(__float2half_rn(y));
              }
              outp += p.ld_out;
            }
          }
        }
      } else {
        if constexpr (T::kRedInRing) cluster_sync_all();   // every CTA of the cluster is done with its operand ring
        // split-K: push this CTA's partial sums into the CTAs that own the token rows (row j belongs to cluster
        // rank j mod num_splits; slot (j div num_splits) * num_splits + this rank of its buffer).  Remote stores
        // do not stall the way remote loads do, and after the cluster barrier every CTA only reads its own memory.
        const uint32_t my_rank = static_cast<uint32_t>(split);
        const int sh = num_splits == 2 ? 1 : num_splits == 4 ? 2 : 3;   // a tile is shared by 2, 4 or 8 CTAs
        const uint32_t red_base = smem_base + T::kOffRed + row * 4;
#pragma unroll
        for (int t = 0; t < TOK; ++t) {
          const uint32_t slot = (static_cast<uint32_t>(t >> sh) << sh) + my_rank;
          st_dsmem_f32(map_to_cta(red_base + slot * (kTileN * 4), static_cast<uint32_t>(grp_base + (t & (num_splits - 1)))), acc[t]);
        }
      }
    }
  }
  if constexpr (!DUMP && T::kRedInRing) {
    if (num_splits > 1 && warp >= T::kEpiWarps) cluster_sync_all();   // the other warps' share of the barrier above
  }

  if constexpr (!DUMP) {
    if (num_splits > 1) {
      // split-K: fixed-order reduction over the cluster through distributed shared memory.
      // Every thread of the CTA helps: the CTA owns TOK / num_splits token rows of 128 features, and slot
      // k * num_splits + r of the buffer holds rank r's partial sum of row my_rank + k * num_splits.
      const float kScaleDown = 5.62949953421312e14f;
      grid_dep_wait();
      const int my_rank = split;
      const int rows = TOK / num_splits;
      constexpr int kMaxIter = (TOK / 2 * kTileN + T::kThreads - 1) / T::kThreads;
      float xs[kMaxIter];     // the token scales of this thread's outputs, fetched before the barrier
#pragma unroll
      for (int it = 0; it < kMaxIter; ++it) {
        const int idx = threadIdx.x + it * T::kThreads;
        const int m = m0 + my_rank + (idx >> 7) * num_splits;
        xs[it] = (idx < rows * kTileN && m < p.M) ? __ldg(p.x_scale + m) * kScaleDown : 0.f;
      }
      __syncwarp();
      cluster_sync_all();
      if (threadIdx.x == 0) SK_TRACE_EVENT(4, 5);
      {
        const float* red = reinterpret_cast<const float*>(smem + T::kOffRed);
#pragma unroll
        for (int it = 0; it < kMaxIter; ++it) {
          const int idx = threadIdx.x + it * T::kThreads;
          const int k = idx >> 7, row = idx & 127;
          const int m = m0 + my_rank + k * num_splits;
          const int n = n0 + row;
          if (idx < rows * kTileN && m < p.M && n < p.N) {
            const float* src = red + (k * num_splits) * kTileN + row;
            // every load of an output is issued before the first add; the sum runs in rank order (deterministic)
            float sum;
            if (num_splits == 2) {
              const float a0 = src[0], a1 = src[kTileN];
              sum = a0 + a1;
            } else if (num_splits == 4) {
              const float a0 = src[0], a1 = src[kTileN], a2 = src[2 * kTileN], a3 = src[3 * kTileN];
              sum = ((a0 + a1) + a2) + a3;
            } else {
              float a[8];
#pragma unroll
              for (int r = 0; r < 8; ++r) a[r] = src[r * kTileN];
              sum = a[0];
#pragma unroll
              for (int r = 1; r < 8; ++r) sum += a[r];
            }
            const float y = sum * xs[it];
            const uint16_t bits = p.out_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(y))
                                             : __half_as_ushort(__float2half_rn(y));
            reinterpret_cast<uint16_t*>(p.out)[static_cast<size_t>(m) * p.ld_out + n] = bits;
            for (int d = 0; d < p.n_extra; ++d)
              reinterpret_cast<uint16_t*>(p.out_extra[d])[static_cast<size_t>(m) * p.ld_out + n] = bits;
          }
        }
      }
      if (threadIdx.x == 0) SK_TRACE_EVENT(4, 6);
      // no second cluster barrier: after the one above no CTA touches another CTA's shared memory
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
