// The W2A8 GEMM kernel for prefill-sized token counts on sm_100a: a PAIR of CTAs (one thread-block cluster of two,
// on two SMs) computes 256 output features x 256 tokens with tcgen05.mma.cta_group::2.
//
// Why a pair.  The one-CTA kernel (w2a8_umma.cuh) with its 128 x 256 tile is bound by shared-memory bandwidth, not
// by the tensor core: per 128-wide K block a CTA's shared memory takes 36 KB of TMA writes (4 KB of packed weights
// + the 32 KB token tile), 4 KB of reads and 16 KB of writes by the expanders, and 48 KB of operand reads by the
// tensor core (16 KB of weights + the 32 KB token tile) -- ~104 KB against the 64 KB that 512 cycles of MMAs at
// 128 B/clk would allow (measured: shared-memory data pipe ~90 % busy, tensor pipe 53 %).  The token tile is two
// thirds of that, and every CTA working on the same 256 tokens fetches and reads its own copy.  With cta_group::2
// the two CTAs of a pair each hold HALF of the token tile (128 tokens): the pair's MMA reads each half once and feeds
// both tensor cores, so per CTA the TMA writes drop to 20 KB and the operand reads to 32 KB per K block (72 KB in
// all), and the stream from L2 drops by 44 %.  No multicast copy is involved: each CTA's TMA loads write only its
// own shared memory.
//
// Structure per CTA (same roles as the one-CTA kernel):
//   producer     1 warp    bulk copy of the 4 KiB tiled weight block of ITS 128 features + tensor-map TMA of ITS
//                          128 tokens x 128 B of the pair's token tile, into a ring of stages (mbarriers)
//   expanders    4 warps   2-bit -> int8 (byte permute), written into the 128-byte-swizzled K-major layout
//   MMA issuers  2 warps   (CTA of cluster rank 0 only) taking the scale groups in turn: 4 x tcgen05.mma.cta_group::2
//                          .kind::i8 of 256 x 256 x 32 per group; its commits arrive on the barriers of BOTH CTAs
//   epilogue     8 warps   double-buffered tcgen05.ld of the group's accumulator (this CTA's 128 features x 256
//                          tokens), one FFMA per value (summation by parts over running sums, as in the one-CTA
//                          kernel); token scale, conversion, transpose through shared memory, TMA / vector stores
// Hand-overs that gate the MMAs live in the shared memory of the rank-0 CTA: the expander warps and the epilogue
// warps of both CTAs arrive there (the rank-1 CTA with mbarrier.arrive on the mapped cluster address).  An expander
// warp arrives only after it has seen its own stage land, so "all expanders of both CTAs arrived" also says that
// both halves of the token tile are in place.
//
// Replaces the reference's cluster-of-two kernel with multicast (slimkernels/cute/gemm/wgmma_sm90_W2A8.cu:165-424,
// cluster shape :208, :475); shares no code with it.
#pragma once
#include "w2a8_umma.cuh"

namespace sk {

// ---------------------------------------------------------------- PTX used only by the pair kernel
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_slot, uint32_t ncols) {   // one warp in EACH CTA of the pair
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem of both CTAs] (+)= A[smem of each CTA: its 128 rows] * B[smem: each CTA holds half of the N rows]^T
__device__ __forceinline__ void umma_i8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives (count 1) on the barrier at this shared-memory offset in BOTH CTAs of the pair once every tcgen05 operation
// issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile(
      "{\n\t.reg .b16 m;\n\t"
      "mov.b16 m, 3;\n\t"
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n\t}"
      ::"r"(bar)
      : "memory");
}
// One arrival on a barrier that lives in the shared memory of the CTA of cluster rank `rank` (may be this CTA).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar, uint32_t rank) {
  asm volatile(
      "{\n\t.reg .b32 r;\n\t"
      "mapa.shared::cluster.u32 r, %0, %1;\n\t"
      "mbarrier.arrive.shared::cluster.b64 _, [r];\n\t}"
      ::"r"(bar), "r"(rank)
      : "memory");
}
// The same without release semantics, for hand-overs that carry no memory written by this thread: an epilogue warp
// handing an accumulator buffer back has only READ tensor memory, and the tcgen05 fences on either side of the
// barrier order those reads before the MMAs that follow.  (A cluster-scope release costs about a thousand cycles.)
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t bar, uint32_t rank) {
  asm volatile(
      "{\n\t.reg .b32 r;\n\t"
      "mapa.shared::cluster.u32 r, %0, %1;\n\t"
      "mbarrier.arrive.shared::cluster.b64 _, [r];\n\t}"
      ::"r"(bar), "r"(rank)
      : "memory");
}
// Bounded wait on a barrier whose arrivals may come from the other CTA of the pair: the polls are the ordinary
// CTA-scope ones (a cluster-scope acquire on every poll is far more expensive), and one cluster-scope fence after
// the phase has been seen complete orders what follows behind the other CTA's released writes.
__device__ __forceinline__ bool wait_bounded_cluster(uint32_t bar, uint32_t parity, const WaitCtx& ctx, int code) {
  const bool ok = wait_bounded(bar, parity, ctx, code);
  asm volatile("fence.acq_rel.cluster;" ::: "memory");
  return ok;
}

template <int STAGES>
struct PairTraits {
  static constexpr int kTokens = 256;                 // tokens of the pair's tile (MMA N)
  static constexpr int kHalfTokens = 128;             // tokens each CTA loads
  static constexpr int kAccBufs = 2;                  // 2 x 256 columns: all of tensor memory
  static constexpr int kEpiWgs = 2, kEpiWarps = 8, kEpiThreads = 256, kExpWarps = 4;
  static constexpr int kThreads = 512;                // 8 epilogue + 4 expander + producer + 2 MMA warps, + 1 idle
  static constexpr int kCols = kTokens / kEpiWgs;     // 128 accumulators per epilogue thread
  static constexpr int kChunk = 32, kNumChunks = kCols / kChunk;
  static constexpr uint32_t kTmemCols = 512;
  static constexpr int kXBytes = kHalfTokens * kBlockK;                 // 16 KB
  static constexpr int kOffX = 0;
  static constexpr int kOffWx = kOffX + STAGES * kXBytes;
  static constexpr int kOffWp = kOffWx + STAGES * kWxBytes;
  static constexpr int kOffBar = kOffWp + STAGES * kWpBytes;
  static constexpr int kNumBars = 3 * STAGES + 2 * kAccBufs;
  static constexpr int kOffMisc = kOffBar + kNumBars * 8;
  static constexpr int kOffXs = kOffMisc + 16;                          // fp32 [256]: x_scale * 2^49 of the tile's tokens
  static constexpr int kTotal = kOffXs + kTokens * 4;
  static constexpr int kDynamicBytes = kTotal + 1024;
  static_assert(kTokens * kTileN * 2 <= kOffBar, "output staging must fit in the operand ring");
  static_assert(kDynamicBytes <= 227 * 1024, "shared memory");
  // register budgets after setmaxnreg (the CTA's pool is 512 threads x 128): epilogue 224, expanders 32, control 32
  static constexpr int kEpiRegs = 224, kExpRegs = 32, kCtlRegs = 32;
  static_assert(kEpiThreads * kEpiRegs + 128 * kExpRegs + 128 * kCtlRegs <= kThreads * 128, "setmaxnreg budgets");
};

template <int STAGES, bool DUMP>
__global__ void __launch_bounds__(PairTraits<STAGES>::kThreads, 1)
w2a8_pair_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_out,
                 const __grid_constant__ ExtraOutMaps tmap_extra, const GemmParams p) {
  using T = PairTraits<STAGES>;
  constexpr int kChunk = T::kChunk, kNumChunks = T::kNumChunks, kCols = T::kCols;
  constexpr int BLOCK_M = T::kTokens, ACC_BUFS = T::kAccBufs;
  constexpr uint32_t kStageTxBytes = kWpBytes + T::kXBytes;
  constexpr int kExpWarp0 = T::kEpiWarps;
  constexpr int kProducerWarp = kExpWarp0 + T::kExpWarps;
  constexpr int kMmaWarp = kProducerWarp + 1;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_ld_full = smem_base + T::kOffBar;          // [STAGES] this CTA's copies of a stage have landed (local)
  const uint32_t bar_ld_empty = bar_ld_full + 8u * STAGES;      // [STAGES] the MMAs that read the stage are complete (commit, both CTAs)
  const uint32_t bar_ex_full = bar_ld_empty + 8u * STAGES;      // [STAGES] rank 0 only: expanded weights of BOTH CTAs are in place
  const uint32_t bar_acc_full = bar_ex_full + 8u * STAGES;      // [ACC_BUFS] the MMAs of a group are complete (commit, both CTAs)
  const uint32_t bar_acc_empty = bar_acc_full + 8u * ACC_BUFS;  // [ACC_BUFS] rank 0 only: BOTH epilogues have read the buffer
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + T::kOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + T::kOffMisc + 4);
  const WaitCtx ctx{abort_flag, p.status, p.wait_limit};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();             // 0: issues the pair's MMAs
  // pairs are numbered like the tiles of the one-CTA kernel (bands of four token tiles), two feature tiles per pair
  const int n_pairs = p.n_tiles >> 1;
  const int pair = static_cast<int>(blockIdx.x >> 1) + static_cast<int>(blockIdx.y) * n_pairs;
  const TileCoord tc = tile_coord(pair, n_pairs, p.num_tiles >> 1);
  const int n_tile = 2 * tc.n_tile + static_cast<int>(rank);
  const int n0 = n_tile * kTileN;
  const int m0 = tc.m_tile * BLOCK_M;
  const int kb_end = p.groups;                         // group size 128: one K block per scale group
  const uint32_t bias = 1u << 22;

  // ---------------------------------------------------------------- set-up
  if (threadIdx.x == 0) SK_TRACE_EVENT(4, 0);
  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(bar_ld_full + 8 * i, 1);                        // TMA transaction bytes
      mbar_init(bar_ld_empty + 8 * i, 1);                       // one commit
      mbar_init(bar_ex_full + 8 * i, 2 * T::kExpWarps);         // expander warps of both CTAs
    }
    for (int i = 0; i < ACC_BUFS; ++i) {
      mbar_init(bar_acc_full + 8 * i, 1);
      mbar_init(bar_acc_empty + 8 * i, 2 * T::kEpiWarps);       // epilogue warps of both CTAs
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == kProducerWarp && lane == 0) prefetch_tensormap(&tmap_x);
  if (warp == kMmaWarp) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), T::kTmemCols);
    tmem_relinquish_pair();
  }
  tcgen05_fence_before_sync();
  cluster_sync_all();            // the barriers of both CTAs exist before anybody arrives on the other CTA's
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp >= kExpWarp0) {
    if (warp < kProducerWarp) setmaxnreg_dec<T::kExpRegs>(); else setmaxnreg_dec<T::kCtlRegs>();
    if (warp == kProducerWarp) {
      // ============================================================ producer (whole warp loops, one lane issues)
      const uint8_t* wsrc = p.w_tiled + static_cast<size_t>(n_tile) * p.k_blocks * kWpBytes;
      const int mx = m0 + static_cast<int>(rank) * T::kHalfTokens;    // this CTA's half of the token tile
      int stage = 0, issued = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = 0; kb < kb_end; ++kb) {
        ok = wait_bounded_relaxed(bar_ld_empty + 8 * stage, phase ^ 1, ctx, kStProducerEmpty, 100);
        if (!ok) break;
        if (elect_one() && kb != p.fault_skip_kb) {
          SK_TRACE_EVENT(0, kb);
          const uint32_t full = bar_ld_full + 8 * stage;
          mbar_arrive_expect_tx(full, kStageTxBytes);
          bulk_load_1d(smem_base + T::kOffWp + stage * kWpBytes, wsrc, kWpBytes, full);
          tma_load_2d(smem_base + T::kOffX + stage * T::kXBytes, &tmap_x, kb * kBlockK, mx, full);
        }
        __syncwarp();
        wsrc += kWpBytes; ++issued;
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
      if (!ok) {
        // Gave up: wait (bounded) until every copy this warp started has landed
        const long long t0 = clock64();
        const int first = issued > STAGES ? issued - STAGES : 0;
        for (int i = first; i < issued; ++i) {
          if (i == p.fault_skip_kb) continue;
          while (!mbar_try_wait(bar_ld_full + 8 * (i % STAGES), (i / STAGES) & 1)) {
            if (clock64() - t0 > ctx.limit) { atomicCAS(p.status, 0, kStDrain); break; }
          }
        }
      }
      __syncwarp();
    } else if ((warp == kMmaWarp || warp == kMmaWarp + 1) && rank == 0) {
      // ============================================================ MMA issuers of the pair (rank 0): two warps take
      // the scale groups in turn, as in the one-CTA kernel
      const int mma_id = warp - kMmaWarp;
      constexpr uint32_t idesc = make_idesc_i8(2 * kTileN, BLOCK_M, /*a_signed=*/true, /*b_signed=*/true);
      const uint64_t a_desc0 = make_kmajor_sw128_desc(smem_base + T::kOffWx);
      const uint64_t b_desc0 = make_kmajor_sw128_desc(smem_base + T::kOffX);
      int l = 0, ab = 0;
      uint32_t lph = 0, aph = 0;
      bool ok = true;
      for (int kb = 0; kb < kb_end; ++kb) {
        if ((kb & 1) == mma_id) {
          if (lane == 0 && kb < 8) SK_TRACE_EVENT(5, kb * 8 + 0);
          ok = wait_bounded_cluster(bar_ex_full + 8 * l, lph, ctx, kStMmaExFull);
          if (lane == 0 && kb < 8) SK_TRACE_EVENT(5, kb * 8 + 1);
          ok = ok && wait_bounded_cluster(bar_acc_empty + 8 * ab, aph, ctx, kStMmaAccEmpty);
          if (lane == 0 && kb < 8) SK_TRACE_EVENT(5, kb * 8 + 2);
          if (!ok) break;
          tcgen05_fence_after_sync();
          if (elect_one()) {
            const uint64_t a_desc = a_desc0 + static_cast<uint64_t>(l * (kWxBytes >> 4));
            const uint64_t b_desc = b_desc0 + static_cast<uint64_t>(l * (T::kXBytes >> 4));
            const uint32_t d = tmem_base + ab * BLOCK_M;
            // +2 in the (address >> 4) field advances 32 bytes along K inside the 128-byte swizzle row
            umma_i8_pair(d, a_desc, b_desc, idesc, 1u);
            umma_i8_pair(d, a_desc + 2, b_desc + 2, idesc, 1u);
            umma_i8_pair(d, a_desc + 4, b_desc + 4, idesc, 1u);
            umma_i8_pair(d, a_desc + 6, b_desc + 6, idesc, 1u);
            if (kb < 8) SK_TRACE_EVENT(5, kb * 8 + 3);
            umma_commit_pair(bar_acc_full + 8 * ab);
            if (kb < 8) SK_TRACE_EVENT(5, kb * 8 + 4);
            umma_commit_pair(bar_ld_empty + 8 * l);
            SK_TRACE_EVENT(2, kb);
          }
          __syncwarp();
        }
        if (++l == STAGES) { l = 0; lph ^= 1; }
        if (++ab == ACC_BUFS) { ab = 0; aph ^= 1; }
      }
      __syncwarp();
    } else if (warp < kProducerWarp) {
      // ============================================================ expanders (one weight row per thread)
      const int row = threadIdx.x - kExpWarp0 * 32;
      const int zp = p.zero_point;
      const uint32_t lut = (static_cast<uint32_t>(0 - zp) & 0xffu) | ((static_cast<uint32_t>(1 - zp) & 0xffu) << 8) |
                           ((static_cast<uint32_t>(2 - zp) & 0xffu) << 16) | ((static_cast<uint32_t>(3 - zp) & 0xffu) << 24);
      // Row r of the expanded tile lives at r * 128; its 16-byte chunk c sits at chunk (c ^ (r & 7))
      const uint32_t wx_off = T::kOffWx + row * 128 + ((row & 7) << 4);
      const uint32_t wp_off = T::kOffWp + row * 16;
      int l = 0;
      uint32_t lph = 0;
      for (int kb = 0; kb < kb_end; ++kb) {
        // The loads below must not be issued before the wait has been seen to succeed.  The stage's previous expanded
        // weights are free: the producer refilled the stage only after the commit of the MMAs that read them.
        if (threadIdx.x == kExpWarp0 * 32 && kb < 12) SK_TRACE_EVENT(6, kb * 4 + 0);
        if (!wait_bounded(bar_ld_full + 8 * l, lph, ctx, kStExpanderFull)) break;
        if (threadIdx.x == kExpWarp0 * 32 && kb < 12) SK_TRACE_EVENT(6, kb * 4 + 1);
        const uint32_t wp = smem_base + wp_off + l * kWpBytes;
        const uint4 q0 = ld_shared_v4(wp);
        const uint4 q1 = ld_shared_v4(wp + 2048);
        const uint32_t wx = smem_base + wx_off + l * kWxBytes;
        const uint32_t words[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int c = 0; c < 8; ++c) st_shared_v4(wx ^ (c << 4), expand16(words[c], lut));
        fence_proxy_async_smem();   // generic-proxy stores -> visible to the tensor cores' async proxy
        __syncwarp();
        if (threadIdx.x == kExpWarp0 * 32 && kb < 12) SK_TRACE_EVENT(6, kb * 4 + 2);
        // this warp has seen its CTA's stage land (weights AND this CTA's half of the token tile) and has expanded
        if (lane == 0) mbar_arrive_cluster(bar_ex_full + 8 * l, 0);
        if (threadIdx.x == kExpWarp0 * 32) SK_TRACE_EVENT(1, kb);
        if (++l == STAGES) { l = 0; lph ^= 1; }
      }
    }
  } else {
    // ============================================================ epilogue
    setmaxnreg_inc<T::kEpiRegs>();
    const int wg = warp >> 2;
    const int row = (warp & 3) * 32 + lane;      // output feature within the tile == TMEM lane
    const int col0 = wg * kCols;                 // first token column of this thread
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + col0;
    const float kScaleUp = 1.2676506002282294e30f;     // 2^100
    const float bias_f = __uint_as_float(bias);        // bias * 2^-149
    const int n = n0 + row;
    const bool n_ok = n < p.N;

    // pre-set both accumulator buffers to the bias and hand them to the pair's MMA issuer
#pragma unroll
    for (int a = 0; a < ACC_BUFS; ++a) {
#pragma unroll
      for (int c = 0; c < kNumChunks; ++c) tmem_st_fill_32x32(lane_addr + a * BLOCK_M + c * kChunk, bias);
    }
    tmem_st_wait();
    tcgen05_fence_before_sync();
    __syncwarp();
    if (lane == 0) {
#pragma unroll
      for (int a = 0; a < ACC_BUFS; ++a) mbar_arrive_cluster_relaxed(bar_acc_empty + 8 * a, 0);
    }

    float acc[kCols];
#pragma unroll
    for (int j = 0; j < kCols; ++j) acc[j] = 0.f;

    // group scales in a register ring (raw fp16 bits), loaded one group ahead; rows pulled into L2 further ahead
    const unsigned short* sp = reinterpret_cast<const unsigned short*>(p.w_scale) + (n_ok ? n : 0);
    int g_load = 0;
    auto load_scale = [&]() -> unsigned short {
      const unsigned short r = (n_ok && g_load < kb_end) ? __ldg(sp) : static_cast<unsigned short>(0);
      if (g_load + kScalePrefetchGroups < kb_end)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(sp + static_cast<size_t>(kScalePrefetchGroups) * p.N));
      sp += p.N; ++g_load;
      return r;
    };
    for (int i = ACC_BUFS + 1; i < kScalePrefetchGroups && i < kb_end; ++i)
      asm volatile("prefetch.global.L2 [%0];" ::"l"(sp + static_cast<size_t>(i) * p.N));
    unsigned short sr[ACC_BUFS + 1];
#pragma unroll
    for (int i = 0; i <= ACC_BUFS; ++i) sr[i] = load_scale();
    float s_sum = 0.f;
    int flush = 0, ab = 0;
    uint32_t aph = 0;
    bool epi_ok = true;
    constexpr bool kDB = !DUMP;
    constexpr int kBufMask = kDB ? 1 : 0;
    uint32_t v[kBufMask + 1][kChunk];
#pragma unroll 1
    for (int g = 0; g < kb_end && epi_ok; ++g) {
      const float s2 = (__half2float(__ushort_as_half(sr[0])) - __half2float(__ushort_as_half(sr[ACC_BUFS]))) * kScaleUp;
#pragma unroll
      for (int i = 0; i < ACC_BUFS; ++i) sr[i] = sr[i + 1];
      sr[ACC_BUFS] = load_scale();
      const uint32_t buf = lane_addr + ab * BLOCK_M;
      if (threadIdx.x == 0 && g < 8) SK_TRACE_EVENT(7, g * 8 + 0);
      epi_ok = wait_bounded(bar_acc_full + 8 * ab, aph, ctx, kStEpilogueAccFull);   // arrival: the pair's commit
      if (!epi_ok) break;
      if (threadIdx.x == 0 && g < 8) SK_TRACE_EVENT(7, g * 8 + 1);
      tcgen05_fence_after_sync();
      if constexpr (kDB) tmem_ld_32x32(buf, v[0]);
#pragma unroll
      for (int c = 0; c < kNumChunks; ++c) {
        if constexpr (!kDB) tmem_ld_32x32(buf + c * kChunk, v[0]);
        tmem_ld_wait();
        if constexpr (kDB) {
          if (c + 1 < kNumChunks) tmem_ld_32x32(buf + (c + 1) * kChunk, v[(c + 1) & kBufMask]);
        }
        if (c == kNumChunks - 1) {   // buffer fully read: hand it back to the MMA issuer (it keeps accumulating)
          tcgen05_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster_relaxed(bar_acc_empty + 8 * ab, 0);
          if (threadIdx.x == 0 && g < 8) SK_TRACE_EVENT(7, g * 8 + 2);
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
      if (threadIdx.x == 0) SK_TRACE_EVENT(3, g);
      s_sum += s2;
      if (++flush == kBiasFlushGroups) {
        const float corr = s_sum * bias_f;
#pragma unroll
        for (int j = 0; j < kCols; ++j) acc[j] -= corr;
        s_sum = 0.f; flush = 0;
      }
      if (++ab == ACC_BUFS) { ab = 0; aph ^= 1; }
    }
    {
      const float corr = s_sum * bias_f;
#pragma unroll
      for (int j = 0; j < kCols; ++j) acc[j] -= corr;
    }

    // ---------------------------------------------------------------- output
    if constexpr (!DUMP) {
      const float kScaleDown = 5.62949953421312e14f;   // 2^49: acc holds (sum_g s P) * 2^-49
      // The operand ring is dead once the last group has been read (all MMAs and all TMA loads of this CTA are
      // complete; the other CTA's tensor core read this CTA's token half only through those same MMAs): reuse it to
      // transpose the tile.  All epilogue threads must be past their last TMEM read first.
      float* xs_s = reinterpret_cast<float*>(smem + T::kOffXs);
      for (int j = threadIdx.x; j < BLOCK_M; j += T::kEpiThreads)
        xs_s[j] = (m0 + j < p.M) ? __ldg(p.x_scale + m0 + j) * kScaleDown : 0.f;
      named_barrier_sync(1, T::kEpiThreads);
      uint16_t* st = reinterpret_cast<uint16_t*>(smem);   // [256][128] in the output dtype
      if (p.out_bf16) stage_tokens<kCols, true>(acc, 0, xs_s + col0, st + col0 * kTileN + row);
      else stage_tokens<kCols, false>(acc, 0, xs_s + col0, st + col0 * kTileN + row);
      if (p.tma_out) fence_proxy_async_smem();
      named_barrier_sync(1, T::kEpiThreads);
      if (p.tma_out) {
        // one TMA store per destination moves the whole staged tile (clipped at the edges of the output)
        if (threadIdx.x == 0) {
          tma_store_2d(&tmap_out, n0, m0, smem_base);
          for (int d = 0; d < p.n_extra; ++d) tma_store_2d(&tmap_extra.map[d], n0, m0, smem_base);
          bulk_commit_group();
          bulk_wait_group_read0();
        }
      } else {
        for (int d = 0; d <= p.n_extra; ++d) {
          uint16_t* outp = reinterpret_cast<uint16_t*>(d == 0 ? p.out : p.out_extra[d - 1]);
          const bool vec_ok = (n0 + kTileN <= p.N) && (p.ld_out % 8 == 0) && ((reinterpret_cast<uintptr_t>(outp) & 15) == 0);
          if (vec_ok) {
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
        }
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  // Neither CTA leaves while the other may still arrive on its barriers or read its shared memory.
  tcgen05_fence_before_sync();
  cluster_sync_all();
  if (warp == kMmaWarp) {
    tcgen05_fence_after_sync();
    tmem_dealloc_pair(tmem_base, T::kTmemCols);
  }
}

}  // namespace sk
