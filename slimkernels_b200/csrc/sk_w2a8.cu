// C ABI of the W2A8 GEMM (declared in include/sk_w2a8.h) plus the small kernels around the main one:
// weight repack / unrepack, and a CUDA-core checker kernel that reads the reference byte layout directly.
#include "../../include/sk_w2a8.h"

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <mutex>
#include <new>
#include <vector>

#include "activation.cuh"
#include "w2a8_umma.cuh"
#include "w2a8_decode.cuh"
#include "w2a8_stream.cuh"
#include "w2a8_pair.cuh"
#include "weight_prep.cuh"

namespace sk {

// ------------------------------------------------------------------------------------------------
// Tiled weight order.  Block (tile T, k-block B) is 4096 bytes at ((T * k_blocks + B) * 4096); inside it the
// 32-bit word for (row r, 16-code chunk c) sits at byte (c / 4) * 2048 + r * 16 + (c % 4) * 4 and holds
//   sum_{j=0..3} sum_{b=0..3} code[n = 128 T + r][k = 128 B + 16 c + 4 j + b] << (4 b + 2 (j & 1) + 16 (j >> 1)),
// i.e. nibble b of each 16-bit half holds two codes whose low 2 bits, after a mask, are byte-permute selectors.
// The source byte for codes 4j..4j+3 of that chunk (matrix_packer order: first code in bits 7:6) is
// w_packed[n][(128 B + 16 c) / 4 + j].
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t tiled_word_from_bytes(const uint8_t (&src)[4]) {
  uint32_t w = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const uint32_t code = (src[j] >> (6 - 2 * b)) & 3u;
      w |= code << (4 * b + 2 * (j & 1) + 16 * (j >> 1));
    }
  }
  return w;
}

__global__ void repack_kernel(const uint8_t* __restrict__ w_packed, uint32_t* __restrict__ w_tiled, long long N,
                              long long K, int k_blocks, long long total_words) {
  const long long row_bytes = K / 4;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total_words;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    // idx enumerates destination words in memory order
    const long long block = idx >> 10;             // 1024 words per 4 KiB block
    const int in_block = static_cast<int>(idx & 1023);
    const int half = in_block >> 9;                // 512 words per half
    const int r = (in_block >> 2) & 127;
    const int c = half * 4 + (in_block & 3);
    const long long T = block / k_blocks, B = block % k_blocks;
    const long long n = T * 128 + r;
    const long long k = B * 128 + 16 * c;
    uint8_t src[4] = {0, 0, 0, 0};
    if (n < N) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (k + 4 * j < K) src[j] = w_packed[n * row_bytes + k / 4 + j];
    }
    w_tiled[idx] = tiled_word_from_bytes(src);
  }
}

__global__ void unrepack_kernel(const uint32_t* __restrict__ w_tiled, uint8_t* __restrict__ w_packed, long long N,
                                long long K, int k_blocks, long long total_words) {
  const long long row_bytes = K / 4;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total_words;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long block = idx >> 10;
    const int in_block = static_cast<int>(idx & 1023);
    const int half = in_block >> 9;
    const int r = (in_block >> 2) & 127;
    const int c = half * 4 + (in_block & 3);
    const long long T = block / k_blocks, B = block % k_blocks;
    const long long n = T * 128 + r;
    const long long k = B * 128 + 16 * c;
    if (n >= N) continue;
    const uint32_t w = w_tiled[idx];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (k + 4 * j >= K) continue;
      uint32_t byte = 0;
#pragma unroll
      for (int b = 0; b < 4; ++b) byte |= ((w >> (4 * b + 2 * (j & 1) + 16 * (j >> 1))) & 3u) << (6 - 2 * b);
      w_packed[n * row_bytes + k / 4 + j] = static_cast<uint8_t>(byte);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// CUDA-core checker kernel.  Reads the reference byte layout (uint8 [N, K/4], first code in bits 7:6)
// directly, so it does not depend on the repack, the tensor-core path or TMA.  One thread per output
// (m, n): 32 consecutive n per warp (x loads are warp-uniform), exact int32 group partials via dp4a,
// fp32 scaling in group order.  Used to cross-check the tcgen05 kernel at sizes the CPU oracle cannot reach.
// ------------------------------------------------------------------------------------------------
__global__ void w2a8_simt_kernel(const int8_t* __restrict__ x_q, long long ld_x, const float* __restrict__ x_scale,
                                 const uint8_t* __restrict__ w_packed, const __half* __restrict__ w_scale,
                                 void* __restrict__ out, long long ld_out, int32_t* __restrict__ partials, int M, int N,
                                 int K, int G, int zero_point, int out_bf16) {
  const int n = blockIdx.x * 32 + threadIdx.x;
  const int m = blockIdx.y * blockDim.y + threadIdx.y;
  if (n >= N || m >= M) return;
  const uint8_t* wrow = w_packed + static_cast<size_t>(n) * (K / 4);
  const int8_t* xrow = x_q + static_cast<size_t>(m) * ld_x;
  const int groups = K / G;
  float acc = 0.f;
  for (int g = 0; g < groups; ++g) {
    int32_t part = 0;
    for (int k = g * G; k < (g + 1) * G; k += 4) {
      const uint32_t b = wrow[k >> 2];
      const int c0 = static_cast<int>((b >> 6) & 3u) - zero_point, c1 = static_cast<int>((b >> 4) & 3u) - zero_point;
      const int c2 = static_cast<int>((b >> 2) & 3u) - zero_point, c3 = static_cast<int>(b & 3u) - zero_point;
      const uint32_t wv = (static_cast<uint32_t>(c0) & 0xffu) | ((static_cast<uint32_t>(c1) & 0xffu) << 8) |
                          ((static_cast<uint32_t>(c2) & 0xffu) << 16) | ((static_cast<uint32_t>(c3) & 0xffu) << 24);
      const int xv = *reinterpret_cast<const int*>(xrow + k);
      part = __dp4a(xv, static_cast<int>(wv), part);
    }
    if (partials) partials[(static_cast<size_t>(g) * M + m) * N + n] = part;
    acc = fmaf(__half2float(w_scale[static_cast<size_t>(g) * N + n]), static_cast<float>(part), acc);
  }
  if (out) {
    const float y = acc * x_scale[m];
    uint16_t* o = reinterpret_cast<uint16_t*>(out) + static_cast<size_t>(m) * ld_out + n;
    *o = out_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(y)) : __half_as_ushort(__float2half_rn(y));
  }
}

// ------------------------------------------------------------------------------------------------
// Launch-floor probe: what a decode-sized launch costs before it moves a byte.  Same grid, cluster, block size,
// dynamic shared memory and launch attributes as the decode kernel would use, and the same fixed work per CTA
// (barrier initialisation, tensor-memory allocation, one CTA barrier, the cluster barrier of the split-K reduction,
// release); no copies, no arithmetic.  A chain of these in a CUDA graph gives the time per launch below which no
// kernel of this geometry can go.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(DecodeTraits<16>::kThreads, 2) launch_floor_kernel(int* sink) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint32_t tmem_slot;
  __shared__ __align__(8) unsigned long long bars[16];
  grid_dep_launch_dependents();
  if (threadIdx.x == 0) {
    for (int i = 0; i < 16; ++i) mbar_init(smem_u32(&bars[i]), 1);
    fence_mbar_init();
  }
  if (threadIdx.x / 32 == 1) {
    tmem_alloc(smem_u32(&tmem_slot), 256);
    tmem_relinquish();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  grid_dep_wait();
  if (gridDim.z > 1) cluster_sync_all();
  if (sink && smem_raw[threadIdx.x] == 0xff && tmem_slot == 0xffffffffu) *sink = 1;   // keeps the dynamic allocation referenced
  tcgen05_fence_before_sync();
  __syncthreads();
  if (threadIdx.x / 32 == 1) {
    tcgen05_fence_after_sync();
    tmem_dealloc(tmem_slot, 256);
  }
}

// ------------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

struct CachedMap {
  const void* ptr;
  long long M, ld;
  int block_m;
  CUtensorMap map;
};

}  // namespace sk

struct sk_w2a8_plan {
  int device = 0;
  long long N = 0, K = 0;
  int G = 128, zero_point = 1, out_dtype = SK_OUT_F16;
  int k_blocks = 0, n_tiles = 0, sm_count = 148;
  const uint8_t* w_rowmajor = nullptr;  // borrowed (may be null when created from a tiled buffer)
  const uint8_t* w_tiled = nullptr;     // owned or borrowed
  uint8_t* w_tiled_owned = nullptr;
  const __half* w_scale = nullptr;      // borrowed
  __half* w_scale_tiled = nullptr;      // device, owned: [n_tiles][k_blocks][128] copy of the scales (group size 128 only)
  int* status = nullptr;                // device, owned
  // balanced-split decode kernel: scratch for the partial sums of tiles shared between CTAs, and their counters
  float* stream_scratch = nullptr;      // device, owned (null: that kernel is not available for this plan)
  int* stream_counters = nullptr;       // device, owned; zero between launches
  int stream_ctas = 0, stream_slots = 0;
  int last_cuda_error = 0;
  int opt_kernel = 0, opt_token_tile = 0, opt_split_k = 0, opt_persistent = 0, opt_pdl = 0, opt_tma_store = 0;
  long long opt_wait_limit = 0;         // 0: the default limit
  int opt_skip_copy = 0;                // failure-path test hook: 1 + index of the K block whose copies are left out
  std::vector<sk::CachedMap> maps;      // small cache of activation tensor maps
  std::mutex mu;
};

namespace sk {

static int cuda_fail(sk_w2a8_plan* plan, cudaError_t e) {
  if (plan) plan->last_cuda_error = static_cast<int>(e);
  (void)cudaGetLastError();
  return e == cudaErrorMemoryAllocation ? SK_ERR_OUT_OF_MEMORY : SK_ERR_CUDA;
}

#ifdef SK_TRACE
static long long* g_trace_buffer = nullptr;
#endif

constexpr size_t kMapCache = 40;   // cached tensor maps per plan (activations and up to 8 output destinations)

struct LaunchChoice {
  int kernel;      // 1 tcgen05 (general), 2 CUDA-core checker, 3 tcgen05 (decode: token tiles 16 / 32, group size 128),
                   // 4 tcgen05 cta_group::2 (pairs of CTAs share a 256-token tile; group size 128, even number of feature tiles),
                   // 5 tcgen05 (decode, one token tile, K range of the whole problem cut into equal CTA ranges)
  int token_tile;  // 16 / 32 / 64 / 128
  int split_k;     // 1 / 2 / 4 / 8
  int persistent;  // 1: one resident set of CTAs walks all tiles
  int ctas;        // CTAs launched
  int mix_tiles1 = 0, mix_split = 0;   // decode kernel 3, mixed launch (see w2a8_decode.cuh); split_k then reports mix_split
};

static LaunchChoice choose(const sk_w2a8_plan* plan, long long M) {
  LaunchChoice c;
  if (plan->opt_token_tile) c.token_tile = plan->opt_token_tile;
  else c.token_tile = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  const bool decode_ok = plan->G == 128 && c.token_tile <= 32;
  // Decode sizes that are one token tile go to the balanced-split kernel (5) when the plan has its scratch buffer;
  // a forced split (SK_OPT_SPLIT_K) or several token tiles go to the kernel that splits over clusters (3).
  const bool stream_ok = decode_ok && M <= c.token_tile && plan->stream_scratch != nullptr && plan->opt_split_k <= 1;
  // Measured on B200 (M = 16): the balanced split wins once every SM has ~64 K blocks or more to stream (70B-class
  // projections: 53 against 70 us on 57344 x 8192); below that its longer tail -- partial sums meet in L2, three
  // global round trips -- costs more than the even load saves.  Its 32-token variant is slower throughout.
  const bool stream_pays = stream_ok && c.token_tile == 16 &&
                           static_cast<long long>(plan->n_tiles) * plan->k_blocks >= 64LL * plan->sm_count;
  c.kernel = plan->opt_kernel ? plan->opt_kernel : (stream_pays ? 5 : decode_ok ? 3 : 1);
  if (c.kernel == 5 && !stream_ok) c.kernel = 3;
  if (c.kernel == 3 && !decode_ok) c.kernel = 1;
  const int groups = static_cast<int>(plan->K / plan->G);
  if (c.kernel == 5) {
    c.split_k = 1;
    c.persistent = 0;
    c.ctas = plan->stream_ctas;
    return c;
  }
  if (plan->opt_split_k) c.split_k = plan->opt_split_k;
  else {
    // Fill the machine in ONE wave: split the K range of a tile over a cluster while the CTAs still fit the
    // resident capacity (2 CTAs per SM for token tiles <= 32, else 1) and every CTA keeps enough groups to
    // amortise its prologue (8 = two pipeline stages of the decode kernel, else 4).
    const long long tiles = plan->n_tiles * ((M + c.token_tile - 1) / c.token_tile);
    const long long capacity = static_cast<long long>(plan->sm_count) * (c.token_tile <= 32 ? 2 : 1);
    const int min_groups = c.kernel == 3 ? 8 : 4;
    int s = 1;
    if (c.token_tile <= 64)
      while (s < 8 && tiles * (2 * s) <= capacity && groups / (2 * s) >= min_groups) s *= 2;
    c.split_k = s;
  }
  if (c.split_k > groups) c.split_k = 1;
  if (c.token_tile > 64) c.split_k = 1;   // the cluster reduction buffer is sized for small token tiles
  // Decode kernel, one token tile, more feature tiles than SMs (but fewer than CTA slots): with one CTA per tile a
  // few SMs carry two whole tiles and everybody waits for them.  Mixed launch instead: one CTA per tile for as many
  // tiles as there are SMs (rounded down to whole clusters of four), the tiles beyond that split 4 ways (or 2 ways,
  // if there are too many for that) so that they spread over the second CTA slot of many SMs in small pieces.
  if (c.kernel == 3 && !plan->opt_split_k && M <= c.token_tile && c.split_k == 1) {
    const int slots = 2 * plan->sm_count;
    const int tiles1 = (plan->sm_count / 4) * 4;
    const int rest = plan->n_tiles - tiles1;
    if (rest > 0 && plan->n_tiles < slots) {
      if (tiles1 + 4 * rest <= slots && groups >= 16) { c.mix_tiles1 = tiles1; c.mix_split = 4; }
      else if ((rest % 2) == 0 && tiles1 + 2 * rest <= slots && groups >= 8) { c.mix_tiles1 = tiles1; c.mix_split = 2; }
      if (c.mix_split) c.split_k = c.mix_split;
    }
  }
  // With more tiles than the machine holds at once, one resident set of CTAs can walk the tiles instead (option
  // SK_OPT_PERSISTENT = 2): the pipeline of the next tile fills while the previous tile is written out through TMA
  // stores.  Measured on B200 it is not reliably faster than one CTA per tile (all CTAs then move in lock-step and
  // hit L2 in bursts), so it is not the default.
  const long long tiles = plan->n_tiles * ((M + c.token_tile - 1) / c.token_tile);
  const long long capacity = static_cast<long long>(plan->sm_count) * (c.token_tile <= 32 ? 2 : 1);
  c.persistent = (plan->opt_persistent == 2 && tiles > capacity) ? 1 : 0;
  if (c.split_k > 1 || (c.token_tile != 128 && c.token_tile != 256)) c.persistent = 0;
  c.ctas = static_cast<int>(c.persistent ? (tiles < capacity ? tiles : capacity) : tiles * c.split_k);
  if (c.mix_split) c.ctas = c.mix_tiles1 + (plan->n_tiles - c.mix_tiles1) * c.mix_split;
  // Pairs of CTAs (cta_group::2) are an option (SK_OPT_KERNEL = 4), not the default: measured on B200 the pair
  // kernel runs at ~1400 TOP/s where one CTA per tile runs at ~2300.  Its MMAs themselves run at full rate (128.8
  // cycles per 256 x 256 x 32), but every hand-over between the two CTAs costs ~290 cycles (remote mbarrier arrival,
  // multicast commit), two of them sit in the cycle MMA -> epilogue -> MMA of each of the two accumulator buffers that
  // fit tensor memory at 256 tokens, and the epilogue is as long as the MMAs of a group.
  const bool pair_ok = c.token_tile == 256 && plan->G == 128 && (plan->n_tiles % 2) == 0 && !c.persistent && c.split_k == 1;
  if (c.kernel == 4 && !pair_ok) c.kernel = 1;
  return c;
}

template <int BLOCK_M, int EPI_WGS, int EXP_WARPS, int LSTAGES, int ESTAGES, int ACC_BUFS, bool DUMP, bool A_TMEM = false,
          bool PERSIST = false>
static int launch_umma(sk_w2a8_plan* plan, const CUtensorMap& map, const CUtensorMap& out_map,
                       const ExtraOutMaps& extra_maps, const GemmParams& prm, int m_tiles, int split_k,
                       int persistent_ctas, cudaStream_t stream) {
  using L = KernelTraits<BLOCK_M, EPI_WGS, EXP_WARPS, LSTAGES, ESTAGES, ACC_BUFS, A_TMEM, PERSIST>;
  auto kern = w2a8_umma_kernel<BLOCK_M, EPI_WGS, EXP_WARPS, LSTAGES, ESTAGES, ACC_BUFS, DUMP, A_TMEM, PERSIST>;
  static int configured_device_mask[64] = {0};
  if (plan->device < 64 && !configured_device_mask[plan->device]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes);
    if (e != cudaSuccess) return cuda_fail(plan, e);
    configured_device_mask[plan->device] = 1;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = PERSIST ? dim3(static_cast<unsigned>(persistent_ctas), 1, 1) : dim3(plan->n_tiles, m_tiles, split_k);
  cfg.blockDim = dim3(L::kThreads, 1, 1);
  cfg.dynamicSmemBytes = L::kDynamicBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (split_k > 1) {
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = split_k;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, map, out_map, extra_maps, prm);
  if (e != cudaSuccess) return cuda_fail(plan, e);
  return SK_OK;
}

template <int TOK, bool DUMP>
static int launch_decode(sk_w2a8_plan* plan, const CUtensorMap& map, const GemmParams& prm, int m_tiles, int split_k,
                         cudaStream_t stream, int mixed_ctas = 0) {
  using L = DecodeTraits<TOK>;
  auto kern = w2a8_decode_kernel<TOK, DUMP>;
  static int configured_device_mask[64] = {0};
  if (plan->device < 64 && !configured_device_mask[plan->device]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes);
    if (e != cudaSuccess) return cuda_fail(plan, e);
    configured_device_mask[plan->device] = 1;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = mixed_ctas > 0 ? dim3(mixed_ctas, 1, 1) : dim3(plan->n_tiles, m_tiles, split_k);
  cfg.blockDim = dim3(L::kThreads, 1, 1);
  cfg.dynamicSmemBytes = L::kDynamicBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (mixed_ctas > 0) {            // clusters of four along x: four single-tile CTAs, or the shares of one or two tiles
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 4;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  } else if (split_k > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = split_k;
    ++na;
  }
  // Programmatic dependent launch: this kernel's set-up and first weight copies may overlap the tail of the previous
  // kernel in the stream (the kernel itself waits for that kernel before it touches activations or outputs, and its
  // roles sit in griddepcontrol.wait rather than poll).  SK_OPT_DEPENDENT_LAUNCH = 1 launches plainly.
  if (!DUMP && plan->opt_pdl != 1) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, map, prm);
  if (e != cudaSuccess) return cuda_fail(plan, e);
  return SK_OK;
}

template <int TOK, int EXP_WARPS>
static int launch_stream(sk_w2a8_plan* plan, const CUtensorMap& map, const GemmParams& prm, cudaStream_t stream) {
  using L = StreamTraits<TOK, EXP_WARPS>;
  auto kern = w2a8_stream_kernel<TOK, EXP_WARPS>;
  static int configured_device_mask[64] = {0};
  if (plan->device < 64 && !configured_device_mask[plan->device]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes);
    if (e != cudaSuccess) return cuda_fail(plan, e);
    configured_device_mask[plan->device] = 1;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(plan->stream_ctas, 1, 1);
  cfg.blockDim = dim3(L::kThreads, 1, 1);
  cfg.dynamicSmemBytes = L::kDynamicBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  int na = 0;
  if (plan->opt_pdl != 1) {   // programmatic dependent launch, as for the other decode kernel
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, map, prm);
  if (e != cudaSuccess) return cuda_fail(plan, e);
  return SK_OK;
}

static int dispatch_stream(sk_w2a8_plan* plan, int token_tile, const CUtensorMap& map, const GemmParams& prm,
                           cudaStream_t stream) {
  // (the kernel can be built with 8 or 16 expander warps and one CTA per SM; measured on B200 that is slower than
  // two CTAs of four expander warps per SM)
  return token_tile == 16 ? launch_stream<16, 4>(plan, map, prm, stream) : launch_stream<32, 4>(plan, map, prm, stream);
}

// Geometry of the balanced-split decode kernel for a plan: how many CTAs, and the most CTAs that share one tile.
// want_ctas = 0: two CTAs per SM, but no CTA with less than one half stage.
static void stream_geometry(const sk_w2a8_plan* plan, int want_ctas, int* ctas_out, int* slots_out) {
  const int units_per_tile = plan->k_blocks / 2;
  const long long units = static_cast<long long>(plan->n_tiles) * units_per_tile;
  long long ctas = want_ctas > 0 ? want_ctas : 2LL * plan->sm_count;
  if (ctas > units) ctas = units;
  int slots = 1;
  for (long long t = 0; t < plan->n_tiles; ++t) {
    const int first = stream_owner(units, static_cast<int>(ctas), t * units_per_tile);
    const int last = stream_owner(units, static_cast<int>(ctas), (t + 1) * units_per_tile - 1);
    if (last - first + 1 > slots) slots = last - first + 1;
  }
  *ctas_out = static_cast<int>(ctas);
  *slots_out = slots;
}

// (Re)allocates the scratch buffer and the counters of the balanced-split decode kernel.  Not on the call path: plan
// creation and sk_w2a8_set_option only.  The device of the plan is current.
static int stream_setup(sk_w2a8_plan* plan, int want_ctas) {
  if (plan->stream_scratch) { cudaFree(plan->stream_scratch); plan->stream_scratch = nullptr; }
  if (plan->stream_counters) { cudaFree(plan->stream_counters); plan->stream_counters = nullptr; }
  plan->stream_ctas = plan->stream_slots = 0;
  if (plan->G != 128 || (plan->K % 256) != 0) return SK_OK;   // whole half stages only: the other decode kernel serves the rest
  int ctas = 0, slots = 0;
  stream_geometry(plan, want_ctas, &ctas, &slots);
  const size_t bytes = static_cast<size_t>(plan->n_tiles) * slots * StreamTraits<32>::kSlotFloats * sizeof(float);
  cudaError_t e = cudaMalloc(&plan->stream_scratch, bytes);
  if (e != cudaSuccess) { plan->stream_scratch = nullptr; return cuda_fail(plan, e); }
  const size_t cbytes = static_cast<size_t>(plan->n_tiles) * StreamTraits<32>::kEpiWarps * sizeof(int);
  e = cudaMalloc(&plan->stream_counters, cbytes);
  if (e == cudaSuccess) e = cudaMemset(plan->stream_counters, 0, cbytes);
  if (e != cudaSuccess) {
    cudaFree(plan->stream_scratch);
    plan->stream_scratch = nullptr;
    if (plan->stream_counters) { cudaFree(plan->stream_counters); plan->stream_counters = nullptr; }
    return cuda_fail(plan, e);
  }
  plan->stream_ctas = ctas;
  plan->stream_slots = slots;
  return SK_OK;
}

constexpr int kPairStages = 6;

template <bool DUMP>
static int launch_pair(sk_w2a8_plan* plan, const CUtensorMap& map, const CUtensorMap& out_map,
                       const ExtraOutMaps& extra_maps, const GemmParams& prm, int m_tiles, cudaStream_t stream) {
  using L = PairTraits<kPairStages>;
  auto kern = w2a8_pair_kernel<kPairStages, DUMP>;
  static int configured_device_mask[64] = {0};
  if (plan->device < 64 && !configured_device_mask[plan->device]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes);
    if (e != cudaSuccess) return cuda_fail(plan, e);
    configured_device_mask[plan->device] = 1;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(plan->n_tiles, m_tiles, 1);
  cfg.blockDim = dim3(L::kThreads, 1, 1);
  cfg.dynamicSmemBytes = L::kDynamicBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;      // the two CTAs of a pair: adjacent feature tiles, same token tile
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, map, out_map, extra_maps, prm);
  if (e != cudaSuccess) return cuda_fail(plan, e);
  return SK_OK;
}

constexpr int kAccBufsSmall = 4;   // accumulator buffers of the token tiles <= 128
constexpr int kAccBufs256 = 2;     // 2 x 256 columns fill the tensor memory
static int acc_bufs_of(int token_tile, int kernel) {
  if (kernel == 3 || kernel == 5) return token_tile == 16 ? DecodeTraits<16>::kAccBufs : DecodeTraits<32>::kAccBufs;
  return token_tile >= 192 ? kAccBufs256 : kAccBufsSmall;
}

// The running sum of one accumulator buffer must stay inside (-2^22, 2^22):
// (K handled per buffer) * 127 * max|code - zp| < 2^22.
static bool running_sum_fits(const sk_w2a8_plan* plan, int token_tile, int split_k, int kernel) {
  const long long groups = plan->K / plan->G;
  const long long groups_cta = (groups + split_k - 1) / split_k;
  const int ab = acc_bufs_of(token_tile, kernel);
  const long long k_per_buf = ((groups_cta + ab - 1) / ab) * plan->G;
  const int mx = plan->zero_point > 3 - plan->zero_point ? plan->zero_point : 3 - plan->zero_point;
  return k_per_buf * 127 * mx < (1LL << 22);
}

// The launch run_gemm makes for M tokens: the heuristic choice, then the depth check.  A K range too deep for the two
// accumulator buffers of the 256-token tile falls back to 128 tokens (four buffers, half the depth per buffer);
// beyond that the call is refused.
static int resolve_launch(const sk_w2a8_plan* plan, long long M, bool debug_partials, LaunchChoice* out) {
  LaunchChoice ch = choose(plan, M);
  if (debug_partials) {
    if (ch.kernel == 5) { ch.kernel = 3; ch.ctas = static_cast<int>(plan->n_tiles * ((M + ch.token_tile - 1) / ch.token_tile)); }
    ch.split_k = 1; ch.persistent = 0; ch.mix_tiles1 = ch.mix_split = 0;
  }
  // (mixed launch: the CTAs with a tile of their own run the whole depth)
  if (ch.kernel != 2 && !running_sum_fits(plan, ch.token_tile, ch.mix_split ? 1 : ch.split_k, ch.kernel)) {
    if (ch.token_tile >= 192 && !plan->opt_token_tile && running_sum_fits(plan, 128, 1, 1)) {
      ch.token_tile = 128;
      ch.persistent = 0;
      ch.ctas = static_cast<int>(plan->n_tiles * ((M + 127) / 128));
    } else {
      return SK_ERR_BAD_SHAPE;   // K too deep for the int32 running sums of this tile configuration
    }
  }
  *out = ch;
  return SK_OK;
}

// The scales of a group-size-128 plan in the order the decode kernels stream them: [n_tiles][k_blocks][128 features]
// (rows past N are zero), so that the scales of a CTA's K range are one contiguous run.
__global__ void tile_scales_kernel(const __half* __restrict__ w_scale, __half* __restrict__ tiled, long long N,
                                   int k_blocks, long long total) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i % kTileN);
    const long long t = i / kTileN;
    const int kb = static_cast<int>(t % k_blocks);
    const long long n = (t / k_blocks) * kTileN + r;
    tiled[i] = n < N ? w_scale[static_cast<size_t>(kb) * N + n] : __float2half(0.f);
  }
}


// Test aid: the expander's shared-memory image of one 128 x 128 weight block next to the image the TMA writes for the
// same int8 values.  One CTA: (a) copies a 4 KiB tiled block into shared memory and expands it exactly as the general
// kernel's expander threads do (expand16, one row per thread, 16-byte stores into the 128-byte-swizzled K-major
// layout); (b) loads the pre-expanded row-major int8 block through a tensor map with CU_TENSOR_MAP_SWIZZLE_128B -- the
// layout the MMA's shared-memory descriptor expects of both operands; (c) writes both 16 KiB images out and counts
// the bytes that differ.  The wait for the TMA is bounded.
__global__ void __launch_bounds__(128)
expander_image_kernel(const __grid_constant__ CUtensorMap tmap_expanded, const uint8_t* __restrict__ w_tiled_block,
                      int zero_point, uint8_t* __restrict__ image_expander, uint8_t* __restrict__ image_tma,
                      int* __restrict__ mismatches, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* wp = smem;                        // [4096] tiled 2-bit block
  uint8_t* wx = smem + 4096;                 // [16384] expander image (1024-aligned: 4096 is)
  uint8_t* wt = smem + 4096 + kWxBytes;      // [16384] TMA image
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_flag;
  const uint32_t bar_a = smem_u32(&bar);
  const int row = threadIdx.x;
  if (threadIdx.x == 0) {
    mbar_init(bar_a, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  for (int i = threadIdx.x; i < kWpBytes / 16; i += blockDim.x)
    reinterpret_cast<uint4*>(wp)[i] = reinterpret_cast<const uint4*>(w_tiled_block)[i];
  __syncthreads();
  if (threadIdx.x == 0) {
    mbar_arrive_expect_tx(bar_a, kWxBytes);
    tma_load_2d(smem_u32(wt), &tmap_expanded, 0, 0, bar_a);
  }
  // (a) as the expander threads of w2a8_umma_kernel, one row per thread
  const uint32_t lut = (static_cast<uint32_t>(0 - zero_point) & 0xffu) | ((static_cast<uint32_t>(1 - zero_point) & 0xffu) << 8) |
                       ((static_cast<uint32_t>(2 - zero_point) & 0xffu) << 16) | ((static_cast<uint32_t>(3 - zero_point) & 0xffu) << 24);
  const uint32_t src = smem_u32(wp) + row * 16;
  const uint4 q0 = ld_shared_v4(src);
  const uint4 q1 = ld_shared_v4(src + 2048);
  const uint32_t words[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
  const uint32_t dst = smem_u32(wx) + row * 128 + ((row & 7) << 4);
#pragma unroll
  for (int c = 0; c < 8; ++c) st_shared_v4(dst ^ (c << 4), expand16(words[c], lut));
  // (b) the TMA image
  const WaitCtx ctx{&abort_flag, status, 200000000ll};
  const bool ok = wait_bounded(bar_a, 0, ctx, kStExpanderFull);
  __syncthreads();
  if (!ok) return;
  // (c)
  int bad = 0;
  for (int i = threadIdx.x; i < kWxBytes / 16; i += blockDim.x) {
    const uint4 a = reinterpret_cast<const uint4*>(wx)[i], b = reinterpret_cast<const uint4*>(wt)[i];
    reinterpret_cast<uint4*>(image_expander)[i] = a;
    reinterpret_cast<uint4*>(image_tma)[i] = b;
    const uint32_t x[4] = {a.x ^ b.x, a.y ^ b.y, a.z ^ b.z, a.w ^ b.w};
#pragma unroll
    for (int j = 0; j < 4; ++j)
      for (int k = 0; k < 4; ++k) bad += ((x[j] >> (8 * k)) & 0xffu) ? 1 : 0;
  }
  if (bad) atomicAdd(mismatches, bad);
}

// partials[g] holds the running sum of its accumulator buffer; turn it into the group's own partial sum.
__global__ void diff_partials_kernel(int32_t* __restrict__ partials, int groups, long long mn, int acc_bufs) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < mn;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    for (int g = groups - 1; g >= acc_bufs; --g) partials[g * mn + i] -= partials[(g - acc_bufs) * mn + i];
}

template <bool DUMP>
static int dispatch_umma(sk_w2a8_plan* plan, int token_tile, const CUtensorMap& map, const CUtensorMap& out_map,
                         const ExtraOutMaps& extra_maps, const GemmParams& prm, int m_tiles, int split_k,
                         int persistent_ctas, cudaStream_t stream) {
  switch (token_tile) {
    // <tokens, epilogue warpgroups, expander warps, load stages, expanded stages, accumulator buffers>
    case 16: return launch_umma<16, 1, 8, 4, 4, kAccBufsSmall, DUMP>(plan, map, out_map, extra_maps, prm, m_tiles, split_k, persistent_ctas, stream);
    case 32: return launch_umma<32, 1, 4, 4, 4, kAccBufsSmall, DUMP>(plan, map, out_map, extra_maps, prm, m_tiles, split_k, persistent_ctas, stream);
    case 64: return launch_umma<64, 1, 4, 6, 6, kAccBufsSmall, DUMP>(plan, map, out_map, extra_maps, prm, m_tiles, split_k, persistent_ctas, stream);
    case 128:
      if constexpr (!DUMP)
        if (persistent_ctas > 0)
          return launch_umma<128, 2, 4, 4, 4, kAccBufsSmall, false, false, true>(plan, map, out_map, extra_maps, prm, m_tiles, 1, persistent_ctas, stream);
      return launch_umma<128, 2, 4, 4, 4, kAccBufsSmall, DUMP>(plan, map, out_map, extra_maps, prm, m_tiles, split_k, persistent_ctas, stream);
    // 192 tokens: the expanded weights live in tensor memory (2 x 192 accumulator columns + 4 x 32 weight columns;
    // no expanded-weight ring in shared memory, so the load ring is 7 stages deep)
    case 192: return launch_umma<192, 2, 4, 7, 4, kAccBufs256, DUMP, true>(plan, map, out_map, extra_maps, prm, m_tiles, split_k, persistent_ctas, stream);
    case 256:
      if constexpr (!DUMP)
        if (persistent_ctas > 0)
          return launch_umma<256, 2, 4, 4, 2, kAccBufs256, false, false, true>(plan, map, out_map, extra_maps, prm, m_tiles, 1, persistent_ctas, stream);
      return launch_umma<256, 2, 4, 4, 4, kAccBufs256, DUMP>(plan, map, out_map, extra_maps, prm, m_tiles, split_k, persistent_ctas, stream);
    default: return SK_ERR_BAD_ARGUMENT;
  }
}

static int get_x_map(sk_w2a8_plan* plan, const int8_t* x_q, long long M, long long ld_x, int block_m,
                     CUtensorMap* out) {
  std::lock_guard<std::mutex> lock(plan->mu);
  for (const auto& c : plan->maps)
    if (c.ptr == x_q && c.M == M && c.ld == ld_x && c.block_m == block_m) { *out = c.map; return SK_OK; }
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return SK_ERR_CUDA;
  CachedMap cm;
  cm.ptr = x_q; cm.M = M; cm.ld = ld_x; cm.block_m = block_m;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(plan->K), static_cast<cuuint64_t>(M)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld_x)};
  const cuuint32_t box[2] = {128u, static_cast<cuuint32_t>(block_m)};
  const cuuint32_t estr[2] = {1u, 1u};
  CUresult r = enc(&cm.map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(x_q), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { plan->last_cuda_error = static_cast<int>(r); return SK_ERR_CUDA; }
  if (plan->maps.size() >= kMapCache) plan->maps.erase(plan->maps.begin());
  plan->maps.push_back(cm);
  *out = cm.map;
  return SK_OK;
}

// Tensor map of an output buffer for TMA stores: 16-bit elements, [M][N] with row pitch ld_out, boxes of 128
// features x box_rows tokens (the whole tile, or 64-token rounds of the persistent kernel), no swizzle.
static int get_out_map(sk_w2a8_plan* plan, const void* out, long long M, long long ld_out, int box_rows,
                       CUtensorMap* res) {
  std::lock_guard<std::mutex> lock(plan->mu);
  for (const auto& c : plan->maps)
    if (c.ptr == out && c.M == M && c.ld == ld_out && c.block_m == -box_rows) { *res = c.map; return SK_OK; }
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return SK_ERR_CUDA;
  CachedMap cm;
  cm.ptr = out; cm.M = M; cm.ld = ld_out; cm.block_m = -box_rows;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(plan->N), static_cast<cuuint64_t>(M)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld_out) * 2};
  const cuuint32_t box[2] = {128u, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1u, 1u};
  CUresult r = enc(&cm.map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(out), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { plan->last_cuda_error = static_cast<int>(r); return SK_ERR_CUDA; }
  if (plan->maps.size() >= kMapCache) plan->maps.erase(plan->maps.begin());
  plan->maps.push_back(cm);
  *res = cm.map;
  return SK_OK;
}

static int run_gemm(sk_w2a8_plan* plan, long long M, const int8_t* x_q, long long ld_x, const float* x_scale,
                    void* out, long long ld_out, int32_t* partials, cudaStream_t stream,
                    void* const* extra_outs = nullptr, int n_extra = 0, long long scatter_rows = 0,
                    long long scatter_row0 = 0) {
  if (!plan || !x_q) return SK_ERR_NULL_POINTER;
  if (!partials && (!x_scale || !out)) return SK_ERR_NULL_POINTER;
  if (M <= 0 || M > 0x7fffffffLL / 2) return SK_ERR_BAD_SHAPE;
  if (ld_x < plan->K) return SK_ERR_BAD_SHAPE;
  if (!partials && ld_out < plan->N) return SK_ERR_BAD_SHAPE;
  if ((ld_x % 16) != 0 || (reinterpret_cast<uintptr_t>(x_q) & 15) != 0) return SK_ERR_BAD_ALIGNMENT;
  if (out && (reinterpret_cast<uintptr_t>(out) & 1) != 0) return SK_ERR_BAD_ALIGNMENT;

  int cur = -1;
  cudaError_t e = cudaGetDevice(&cur);
  if (e != cudaSuccess) return cuda_fail(plan, e);
  if (cur != plan->device) {
    e = cudaSetDevice(plan->device);
    if (e != cudaSuccess) return cuda_fail(plan, e);
  }
  LaunchChoice ch;
  int rc = resolve_launch(plan, M, partials != nullptr, &ch);
  if (rc != SK_OK) {
    if (cur != plan->device) (void)cudaSetDevice(cur);
    return rc;
  }
  if (scatter_rows > 0 && (ch.kernel != 1 || ch.split_k != 1 || (scatter_rows % ch.token_tile) != 0)) {
    // row scatter is the general kernel's: every token tile must belong to one destination
    if (cur != plan->device) (void)cudaSetDevice(cur);
    return SK_ERR_UNAVAILABLE;
  }
  if (ch.kernel == 2) {
    if (!plan->w_rowmajor || n_extra > 0) rc = SK_ERR_UNAVAILABLE;
    else {
      dim3 block(32, 8, 1);
      dim3 grid(static_cast<unsigned>((plan->N + 31) / 32), static_cast<unsigned>((M + 7) / 8), 1);
      w2a8_simt_kernel<<<grid, block, 0, stream>>>(x_q, ld_x, x_scale, plan->w_rowmajor, plan->w_scale, out, ld_out,
                                                   partials, static_cast<int>(M), static_cast<int>(plan->N),
                                                   static_cast<int>(plan->K), plan->G, plan->zero_point,
                                                   plan->out_dtype == SK_OUT_BF16);
      e = cudaGetLastError();
      if (e != cudaSuccess) rc = cuda_fail(plan, e);
    }
  } else {
    CUtensorMap map;
    rc = get_x_map(plan, x_q, M, ld_x, ch.kernel == 4 ? 128 : ch.token_tile, &map);
    if (rc == SK_OK) {
      GemmParams prm;
      prm.w_tiled = plan->w_tiled;
      prm.w_scale = plan->w_scale;
      prm.w_scale_tiled = plan->w_scale_tiled;
      prm.x_scale = x_scale;
      prm.out = out;
      prm.n_extra = n_extra;
      prm.scatter_rows = static_cast<int>(scatter_rows);
      prm.scatter_row0 = static_cast<int>(scatter_row0);
      for (int i = 0; i < 7; ++i) prm.out_extra[i] = i < n_extra ? extra_outs[i] : nullptr;
      prm.partials = partials;
      prm.status = plan->status;
      prm.ld_out = ld_out;
      prm.M = static_cast<int>(M);
      prm.N = static_cast<int>(plan->N);
      prm.K = static_cast<int>(plan->K);
      prm.k_blocks = plan->k_blocks;
      prm.steps_per_group = plan->G / 32;
      prm.groups = static_cast<int>(plan->K / plan->G);
      prm.zero_point = plan->zero_point;
      prm.out_bf16 = plan->out_dtype == SK_OUT_BF16;
      prm.wait_limit = plan->opt_wait_limit > 0 ? plan->opt_wait_limit : kWaitLimitCycles;
      prm.fault_skip_kb = plan->opt_skip_copy - 1;
      prm.mix_tiles1 = partials ? 0 : ch.mix_tiles1;
      prm.mix_split = partials ? 0 : ch.mix_split;
      prm.stream_scratch = plan->stream_scratch;
      prm.stream_counters = plan->stream_counters;
      prm.stream_slots = plan->stream_slots;
#ifdef SK_TRACE
      prm.trace = g_trace_buffer;
#endif
      const int m_tiles = static_cast<int>((M + ch.token_tile - 1) / ch.token_tile);
      prm.n_tiles = plan->n_tiles;
      prm.num_tiles = plan->n_tiles * m_tiles;
      // The persistent kernel stores through TMA (and 16-byte vectors for further destinations): the output must be
      // 16-byte aligned with a pitch that is a multiple of 8 elements, N a multiple of 8 (the tensor map's extent in
      // bytes), and with further destinations the feature tiles must be whole.
      bool persist = ch.persistent && scatter_rows == 0 && !partials && (ld_out % 8) == 0 && (plan->N % 8) == 0 &&
                     (reinterpret_cast<uintptr_t>(out) & 15) == 0;
      if (persist && n_extra > 0) {
        if (plan->N % 128) persist = false;
        for (int i = 0; i < n_extra; ++i)
          if (reinterpret_cast<uintptr_t>(extra_outs[i]) & 15) persist = false;
      }
      CUtensorMap out_map = map;   // placeholder where the kernel does not use it
      ExtraOutMaps extra_maps;
      for (int i = 0; i < 7; ++i) extra_maps.map[i] = map;
      if (persist) {
        rc = get_out_map(plan, out, M, ld_out, 64, &out_map);
        if (rc != SK_OK) persist = false, rc = SK_OK;
      }
      // One CTA per tile: the staged tile leaves through one TMA store per destination where the buffers allow it
      // (16-byte aligned, pitch a multiple of 8 elements, N a multiple of 8).
      prm.tma_out = 0;
      if (!persist && !partials && (ch.kernel == 1 || ch.kernel == 4) && ch.split_k == 1 && (ld_out % 8) == 0 && (plan->N % 8) == 0 &&
          (reinterpret_cast<uintptr_t>(out) & 15) == 0 && plan->opt_tma_store != 1) {
        // (row scatter: a destination holds scatter_row0 + scatter_rows rows at least; its map is clipped there)
        const long long map_rows = scatter_rows > 0 ? scatter_row0 + scatter_rows : M;
        bool ok = get_out_map(plan, out, map_rows, ld_out, ch.token_tile, &out_map) == SK_OK;
        for (int i = 0; ok && i < n_extra; ++i)
          ok = (reinterpret_cast<uintptr_t>(extra_outs[i]) & 15) == 0 &&
               get_out_map(plan, extra_outs[i], map_rows, ld_out, ch.token_tile, &extra_maps.map[i]) == SK_OK;
        prm.tma_out = ok ? 1 : 0;
      }
      if (m_tiles > 65535) rc = SK_ERR_BAD_SHAPE;
      else if (partials) {
        if (ch.kernel == 3)
          rc = ch.token_tile == 16 ? launch_decode<16, true>(plan, map, prm, m_tiles, 1, stream)
                                   : launch_decode<32, true>(plan, map, prm, m_tiles, 1, stream);
        else if (ch.kernel == 4) rc = launch_pair<true>(plan, map, out_map, extra_maps, prm, m_tiles, stream);
        else rc = dispatch_umma<true>(plan, ch.token_tile, map, out_map, extra_maps, prm, m_tiles, 1, 0, stream);
        if (rc == SK_OK) {
          const long long mn = M * plan->N;
          const int blocks = static_cast<int>(mn / 256 + 1 < 148 * 8 ? mn / 256 + 1 : 148 * 8);
          diff_partials_kernel<<<blocks, 256, 0, stream>>>(partials, prm.groups, mn, acc_bufs_of(ch.token_tile, ch.kernel));
          e = cudaGetLastError();
          if (e != cudaSuccess) rc = cuda_fail(plan, e);
        }
      }
      else if (ch.kernel == 5)
        rc = dispatch_stream(plan, ch.token_tile, map, prm, stream);
      else if (ch.kernel == 3)
        rc = ch.token_tile == 16 ? launch_decode<16, false>(plan, map, prm, m_tiles, ch.split_k, stream, ch.mix_split ? ch.ctas : 0)
                                 : launch_decode<32, false>(plan, map, prm, m_tiles, ch.split_k, stream, ch.mix_split ? ch.ctas : 0);
      else if (ch.kernel == 4) rc = launch_pair<false>(plan, map, out_map, extra_maps, prm, m_tiles, stream);
      else rc = dispatch_umma<false>(plan, ch.token_tile, map, out_map, extra_maps, prm, m_tiles, ch.split_k, persist ? ch.ctas : 0, stream);
    }
  }
  if (cur != plan->device) (void)cudaSetDevice(cur);
  return rc;
}

static int repack_common(bool forward, const uint8_t* src, long long N, long long K, uint8_t* dst,
                         cudaStream_t stream) {
  if (!src || !dst) return SK_ERR_NULL_POINTER;
  if (N <= 0 || K <= 0 || (K % 32) != 0) return SK_ERR_BAD_SHAPE;
  const uint8_t* tiled = forward ? dst : src;
  if ((reinterpret_cast<uintptr_t>(tiled) & 15) != 0) return SK_ERR_BAD_ALIGNMENT;
  const int k_blocks = static_cast<int>((K + 127) / 128);
  const long long n_tiles = (N + 127) / 128;
  const long long total_words = n_tiles * k_blocks * 1024;
  const int threads = 256;
  const long long want = (total_words + threads - 1) / threads;
  const int blocks = static_cast<int>(want < 148 * 16 ? want : 148 * 16);
  if (forward)
    repack_kernel<<<blocks, threads, 0, stream>>>(src, reinterpret_cast<uint32_t*>(dst), N, K, k_blocks, total_words);
  else
    unrepack_kernel<<<blocks, threads, 0, stream>>>(reinterpret_cast<const uint32_t*>(src), dst, N, K, k_blocks,
                                                    total_words);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return SK_ERR_CUDA;
  return SK_OK;
}

}  // namespace sk

// ================================================================================================
// extern "C"
// ================================================================================================
extern "C" {

int sk_w2a8_version(void) { return 100; }

const char* sk_status_string(int status) {
  switch (status) {
    case SK_OK: return "ok";
    case SK_ERR_NULL_POINTER: return "null pointer";
    case SK_ERR_BAD_SHAPE: return "bad shape";
    case SK_ERR_BAD_ALIGNMENT: return "bad alignment";
    case SK_ERR_UNSUPPORTED_ARCH: return "unsupported architecture (needs compute capability 10.x)";
    case SK_ERR_CUDA: return "CUDA error";
    case SK_ERR_DEVICE_TIMEOUT: return "a bounded wait inside a kernel expired";
    case SK_ERR_BAD_ARGUMENT: return "bad argument";
    case SK_ERR_OUT_OF_MEMORY: return "out of device memory";
    case SK_ERR_UNAVAILABLE: return "not available for this plan";
    case SK_ERR_STATIC_SCRATCH_TOO_SMALL:
      return "problem needs more scratch than the library's fixed no-allocation buffer holds";
    default: return "unknown status";
  }
}

int64_t sk_w2a8_tiled_bytes(int64_t N, int64_t K) {
  if (N <= 0 || K <= 0) return 0;
  return ((N + 127) / 128) * ((K + 127) / 128) * 4096;
}

int sk_w2a8_repack(const uint8_t* w_packed, int64_t N, int64_t K, uint8_t* w_tiled, sk_stream_t stream) {
  return sk::repack_common(true, w_packed, N, K, w_tiled, static_cast<cudaStream_t>(stream));
}

int sk_w2a8_unrepack(const uint8_t* w_tiled, int64_t N, int64_t K, uint8_t* w_packed, sk_stream_t stream) {
  return sk::repack_common(false, w_tiled, N, K, w_packed, static_cast<cudaStream_t>(stream));
}

int sk_w2a8_plan_create(sk_w2a8_plan** out, int device, int64_t N, int64_t K, int group_size, int zero_point,
                        const uint8_t* w, int w_layout, const void* w_scale_f16, int out_dtype) {
  if (!out) return SK_ERR_NULL_POINTER;
  *out = nullptr;
  if (!w || !w_scale_f16) return SK_ERR_NULL_POINTER;
  if (N <= 0 || K <= 0 || N > (1LL << 30) || K > (1LL << 30)) return SK_ERR_BAD_SHAPE;
  if (group_size <= 0 || (group_size % 32) != 0 || (K % group_size) != 0 || (K % 32) != 0) return SK_ERR_BAD_SHAPE;
  if (!((group_size % 128) == 0 || (128 % group_size) == 0)) return SK_ERR_BAD_SHAPE;
  if (zero_point < 0 || zero_point > 3) return SK_ERR_BAD_ARGUMENT;
  if (out_dtype != SK_OUT_F16 && out_dtype != SK_OUT_BF16) return SK_ERR_BAD_ARGUMENT;
  if (w_layout != SK_WEIGHT_ROWMAJOR && w_layout != SK_WEIGHT_TILED) return SK_ERR_BAD_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(w_scale_f16) & 1) != 0) return SK_ERR_BAD_ALIGNMENT;
  if (w_layout == SK_WEIGHT_TILED && (reinterpret_cast<uintptr_t>(w) & 15) != 0) return SK_ERR_BAD_ALIGNMENT;

  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess) { (void)cudaGetLastError(); return SK_ERR_CUDA; }
  if (device < 0 || device >= ndev) return SK_ERR_BAD_ARGUMENT;
  int major = 0, sms = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) {
    (void)cudaGetLastError();
    return SK_ERR_CUDA;
  }
  if (major != 10) return SK_ERR_UNSUPPORTED_ARCH;

  sk_w2a8_plan* plan = new (std::nothrow) sk_w2a8_plan();
  if (!plan) return SK_ERR_OUT_OF_MEMORY;
  plan->device = device;
  plan->N = N; plan->K = K; plan->G = group_size; plan->zero_point = zero_point; plan->out_dtype = out_dtype;
  plan->k_blocks = static_cast<int>((K + 127) / 128);
  plan->n_tiles = static_cast<int>((N + 127) / 128);
  plan->sm_count = sms;
  plan->w_scale = static_cast<const __half*>(w_scale_f16);
  plan->maps.reserve(sk::kMapCache + 1);   // the tensor-map cache never grows past kMapCache entries: no host reallocation on the call path

  int cur = -1;
  cudaGetDevice(&cur);
  cudaError_t e = cudaSetDevice(device);
  int rc = SK_OK;
  if (e != cudaSuccess) rc = sk::cuda_fail(plan, e);
  if (rc == SK_OK) {
    e = cudaMalloc(&plan->status, sizeof(int));
    if (e != cudaSuccess) rc = sk::cuda_fail(plan, e);
    else {
      e = cudaMemset(plan->status, 0, sizeof(int));
      if (e != cudaSuccess) rc = sk::cuda_fail(plan, e);
    }
  }
  if (rc == SK_OK) {
    if (w_layout == SK_WEIGHT_TILED) {
      plan->w_tiled = w;
    } else {
      plan->w_rowmajor = w;
      e = cudaMalloc(&plan->w_tiled_owned, static_cast<size_t>(sk_w2a8_tiled_bytes(N, K)));
      if (e != cudaSuccess) rc = sk::cuda_fail(plan, e);
      else {
        rc = sk::repack_common(true, w, N, K, plan->w_tiled_owned, nullptr);
        if (rc == SK_OK) {
          e = cudaDeviceSynchronize();
          if (e != cudaSuccess) rc = sk::cuda_fail(plan, e);
        }
        plan->w_tiled = plan->w_tiled_owned;
      }
    }
  }
  if (rc == SK_OK && group_size == 128) {
    // the decode kernels' copy of the scales (made once, here: later changes of w_scale_f16 are not seen by them)
    const long long total = static_cast<long long>(plan->n_tiles) * plan->k_blocks * sk::kTileN;
    e = cudaMalloc(&plan->w_scale_tiled, static_cast<size_t>(total) * sizeof(__half));
    if (e != cudaSuccess) { plan->w_scale_tiled = nullptr; rc = sk::cuda_fail(plan, e); }
    else {
      const int blocks = static_cast<int>(total / 256 + 1 < 148 * 8 ? total / 256 + 1 : 148 * 8);
      sk::tile_scales_kernel<<<blocks, 256>>>(plan->w_scale, plan->w_scale_tiled, N, plan->k_blocks, total);
      e = cudaGetLastError();
      if (e == cudaSuccess) e = cudaDeviceSynchronize();
      if (e != cudaSuccess) rc = sk::cuda_fail(plan, e);
    }
  }
  // The balanced-split decode kernel's scratch is allocated here only where that kernel is the default (large weight
  // matrices, see choose()); elsewhere on request (SK_OPT_KERNEL = 5 / SK_OPT_STREAM_CTAS, set-up calls).
  if (rc == SK_OK && static_cast<long long>(plan->n_tiles) * plan->k_blocks >= 64LL * plan->sm_count)
    rc = sk::stream_setup(plan, 0);
  if (cur >= 0 && cur != device) (void)cudaSetDevice(cur);
  if (rc != SK_OK) {
    if (plan->status) cudaFree(plan->status);
    if (plan->w_tiled_owned) cudaFree(plan->w_tiled_owned);
    if (plan->stream_scratch) cudaFree(plan->stream_scratch);
    if (plan->stream_counters) cudaFree(plan->stream_counters);
    if (plan->w_scale_tiled) cudaFree(plan->w_scale_tiled);
    delete plan;
    return rc;
  }
  *out = plan;
  return SK_OK;
}

int sk_w2a8_plan_destroy(sk_w2a8_plan* plan) {
  if (!plan) return SK_ERR_NULL_POINTER;
  int cur = -1;
  cudaGetDevice(&cur);
  (void)cudaSetDevice(plan->device);
  if (plan->status) cudaFree(plan->status);
  if (plan->w_tiled_owned) cudaFree(plan->w_tiled_owned);
  if (plan->stream_scratch) cudaFree(plan->stream_scratch);
  if (plan->stream_counters) cudaFree(plan->stream_counters);
  if (plan->w_scale_tiled) cudaFree(plan->w_scale_tiled);
  if (cur >= 0 && cur != plan->device) (void)cudaSetDevice(cur);
  delete plan;
  return SK_OK;
}

int sk_w2a8_plan_info(const sk_w2a8_plan* plan, int64_t* N, int64_t* K, int* group_size, int* zero_point,
                      int* out_dtype, int* device) {
  if (!plan) return SK_ERR_NULL_POINTER;
  if (N) *N = plan->N;
  if (K) *K = plan->K;
  if (group_size) *group_size = plan->G;
  if (zero_point) *zero_point = plan->zero_point;
  if (out_dtype) *out_dtype = plan->out_dtype;
  if (device) *device = plan->device;
  return SK_OK;
}

int sk_w2a8_set_option(sk_w2a8_plan* plan, int key, int64_t value) {
  if (!plan) return SK_ERR_NULL_POINTER;
  switch (key) {
    case SK_OPT_KERNEL:
      if (value < 0 || value > 5) return SK_ERR_BAD_ARGUMENT;
      if (value == 2 && !plan->w_rowmajor) return SK_ERR_UNAVAILABLE;
      if (value == 5 && !plan->stream_scratch) {   // first request on a plan that did not get the scratch at creation
        int cur = -1;
        cudaGetDevice(&cur);
        (void)cudaSetDevice(plan->device);
        const int rc = sk::stream_setup(plan, 0);
        if (cur >= 0 && cur != plan->device) (void)cudaSetDevice(cur);
        if (rc != SK_OK) return rc;
        if (!plan->stream_scratch) return SK_ERR_UNAVAILABLE;   // group size != 128 or K % 256 != 0
      }
      if (value == 4 && plan->G != 128) return SK_ERR_UNAVAILABLE;
      if (value == 3 && plan->G != 128) return SK_ERR_UNAVAILABLE;
      plan->opt_kernel = static_cast<int>(value);
      return SK_OK;
    case SK_OPT_TOKEN_TILE:
      if (value != 0 && value != 16 && value != 32 && value != 64 && value != 128 && value != 192 && value != 256)
        return SK_ERR_BAD_ARGUMENT;
      plan->opt_token_tile = static_cast<int>(value);
      return SK_OK;
    case SK_OPT_SPLIT_K:
      if (value != 0 && value != 1 && value != 2 && value != 4 && value != 8) return SK_ERR_BAD_ARGUMENT;
      plan->opt_split_k = static_cast<int>(value);
      return SK_OK;
    case SK_OPT_DEPENDENT_LAUNCH:
      if (value < 0 || value > 2) return SK_ERR_BAD_ARGUMENT;
      plan->opt_pdl = static_cast<int>(value);
      return SK_OK;
    case SK_OPT_TMA_STORE:
      if (value < 0 || value > 2) return SK_ERR_BAD_ARGUMENT;
      plan->opt_tma_store = static_cast<int>(value);
      return SK_OK;
    case SK_OPT_PERSISTENT:
      if (value < 0 || value > 2) return SK_ERR_BAD_ARGUMENT;
      plan->opt_persistent = static_cast<int>(value);
      return SK_OK;
    case SK_OPT_WAIT_LIMIT_CYCLES:
      if (value < 0 || (value != 0 && value < 1000)) return SK_ERR_BAD_ARGUMENT;
      plan->opt_wait_limit = value;
      return SK_OK;
    case SK_OPT_STREAM_CTAS: {
      if (value < 0 || value > 65535) return SK_ERR_BAD_ARGUMENT;
      if (plan->G != 128 || (plan->K % 256) != 0) return SK_ERR_UNAVAILABLE;
      int cur = -1;
      cudaGetDevice(&cur);
      (void)cudaSetDevice(plan->device);
      const int rc = sk::stream_setup(plan, static_cast<int>(value));   // frees and allocates: orders itself after the plan's launches
      if (cur >= 0 && cur != plan->device) (void)cudaSetDevice(cur);
      return rc;
    }
    case SK_OPT_TEST_SKIP_COPY:
      if (value < 0 || value > (1 << 20)) return SK_ERR_BAD_ARGUMENT;
      plan->opt_skip_copy = static_cast<int>(value);
      return SK_OK;
    default: return SK_ERR_BAD_ARGUMENT;
  }
}

int sk_w2a8_gemm(sk_w2a8_plan* plan, int64_t M, const int8_t* x_q, int64_t ld_x, const float* x_scale, void* out,
                 int64_t ld_out, sk_stream_t stream) {
  return sk::run_gemm(plan, M, x_q, ld_x, x_scale, out, ld_out, nullptr, static_cast<cudaStream_t>(stream));
}

int sk_w2a8_gemm_scatter(sk_w2a8_plan* plan, int64_t M, const int8_t* x_q, int64_t ld_x, const float* x_scale,
                         void* const* outs, int n_outs, int64_t ld_out, int64_t col_offset, sk_stream_t stream) {
  if (!outs) return SK_ERR_NULL_POINTER;
  if (n_outs < 1 || n_outs > 8) return SK_ERR_BAD_ARGUMENT;
  if (!plan) return SK_ERR_NULL_POINTER;
  if (col_offset < 0 || col_offset + plan->N > ld_out) return SK_ERR_BAD_SHAPE;
  const size_t esz = 2;   // half and bfloat16
  void* shifted[8];
  for (int i = 0; i < n_outs; ++i) {
    if (!outs[i]) return SK_ERR_NULL_POINTER;
    shifted[i] = static_cast<char*>(outs[i]) + static_cast<size_t>(col_offset) * esz;
  }
  return sk::run_gemm(plan, M, x_q, ld_x, x_scale, shifted[0], ld_out, nullptr, static_cast<cudaStream_t>(stream),
                      shifted + 1, n_outs - 1);
}

int sk_w2a8_gemm_rowscatter(sk_w2a8_plan* plan, int64_t M, const int8_t* x_q, int64_t ld_x, const float* x_scale,
                            void* const* outs, int n_outs, int64_t rows_per_dest, int64_t dst_row0, int64_t ld_out,
                            sk_stream_t stream) {
  if (!outs) return SK_ERR_NULL_POINTER;
  if (n_outs < 1 || n_outs > 8) return SK_ERR_BAD_ARGUMENT;
  if (!plan) return SK_ERR_NULL_POINTER;
  if (rows_per_dest <= 0 || dst_row0 < 0 || M != rows_per_dest * n_outs) return SK_ERR_BAD_SHAPE;
  if (dst_row0 + rows_per_dest > 0x7fffffffLL) return SK_ERR_BAD_SHAPE;
  for (int i = 0; i < n_outs; ++i)
    if (!outs[i]) return SK_ERR_NULL_POINTER;
  return sk::run_gemm(plan, M, x_q, ld_x, x_scale, outs[0], ld_out, nullptr, static_cast<cudaStream_t>(stream),
                      outs + 1, n_outs - 1, rows_per_dest, dst_row0);
}

int sk_w2a8_gemm_debug_partials(sk_w2a8_plan* plan, int64_t M, const int8_t* x_q, int64_t ld_x, int32_t* partials,
                                sk_stream_t stream) {
  if (!partials) return SK_ERR_NULL_POINTER;
  return sk::run_gemm(plan, M, x_q, ld_x, nullptr, nullptr, 0, partials, static_cast<cudaStream_t>(stream));
}

int sk_w2a8_last_device_status(sk_w2a8_plan* plan, int* device_status) {
  if (!plan || !device_status) return SK_ERR_NULL_POINTER;
  int cur = -1;
  cudaGetDevice(&cur);
  (void)cudaSetDevice(plan->device);
  int v = 0;
  cudaError_t e = cudaMemcpy(&v, plan->status, sizeof(int), cudaMemcpyDeviceToHost);
  if (e == cudaSuccess && v != 0) e = cudaMemset(plan->status, 0, sizeof(int));
  // a launch that gave up may have left tiles of the balanced-split kernel half counted
  if (e == cudaSuccess && v != 0 && plan->stream_counters)
    e = cudaMemset(plan->stream_counters, 0, static_cast<size_t>(plan->n_tiles) * sk::StreamTraits<32>::kEpiWarps * sizeof(int));
  if (cur >= 0 && cur != plan->device) (void)cudaSetDevice(cur);
  if (e != cudaSuccess) return sk::cuda_fail(plan, e);
  *device_status = v;
  return v == 0 ? SK_OK : SK_ERR_DEVICE_TIMEOUT;
}

int sk_w2a8_last_cuda_error(const sk_w2a8_plan* plan) { return plan ? plan->last_cuda_error : 0; }

int sk_w2a8_launch_floor_probe(sk_w2a8_plan* plan, int64_t M, sk_stream_t stream) {
  if (!plan) return SK_ERR_NULL_POINTER;
  if (M <= 0) return SK_ERR_BAD_SHAPE;
  sk::LaunchChoice ch;
  int rc = sk::resolve_launch(plan, M, false, &ch);
  if (rc != SK_OK) return rc;
  if (ch.kernel != 3 && ch.kernel != 5) return SK_ERR_UNAVAILABLE;   // the probe mirrors the decode kernels' launch
  int cur = -1;
  if (cudaGetDevice(&cur) != cudaSuccess) return sk::cuda_fail(plan, cudaGetLastError());
  if (cur != plan->device && cudaSetDevice(plan->device) != cudaSuccess) return sk::cuda_fail(plan, cudaGetLastError());
  const int dyn = ch.token_tile == 16 ? sk::DecodeTraits<16>::kDynamicBytes : sk::DecodeTraits<32>::kDynamicBytes;
  static int configured[64] = {0};
  cudaError_t e = cudaSuccess;
  if (plan->device < 64 && !configured[plan->device]) {
    e = cudaFuncSetAttribute(sk::launch_floor_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024);
    configured[plan->device] = 1;
  }
  if (e == cudaSuccess) {
    cudaLaunchConfig_t cfg = {};
    const int m_tiles = static_cast<int>((M + ch.token_tile - 1) / ch.token_tile);
    cfg.gridDim = ch.kernel == 5 ? dim3(plan->stream_ctas, 1, 1)
                  : ch.mix_split ? dim3(ch.ctas, 1, 1) : dim3(plan->n_tiles, m_tiles, ch.split_k);
    cfg.blockDim = dim3(sk::DecodeTraits<16>::kThreads, 1, 1);
    cfg.dynamicSmemBytes = dyn - 1024;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (ch.kernel == 3 && ch.mix_split) {
      attr[na].id = cudaLaunchAttributeClusterDimension;
      attr[na].val.clusterDim.x = 4;
      attr[na].val.clusterDim.y = 1;
      attr[na].val.clusterDim.z = 1;
      ++na;
    } else if (ch.kernel == 3 && ch.split_k > 1) {
      attr[na].id = cudaLaunchAttributeClusterDimension;
      attr[na].val.clusterDim.x = 1;
      attr[na].val.clusterDim.y = 1;
      attr[na].val.clusterDim.z = ch.split_k;
      ++na;
    }
    if (plan->opt_pdl != 1) {
      attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[na].val.programmaticStreamSerializationAllowed = 1;
      ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    e = cudaLaunchKernelEx(&cfg, sk::launch_floor_kernel, static_cast<int*>(nullptr));
  }
  if (cur != plan->device) (void)cudaSetDevice(cur);
  return e == cudaSuccess ? SK_OK : sk::cuda_fail(plan, e);
}

const char* sk_device_status_string(int device_status) {
  switch (device_status) {
    case 0: return "no wait expired";
    case sk::kStProducerEmpty: return "producer: a pipeline stage was never released by the MMAs that read it";
    case sk::kStExpanderFull: return "expander: the copies of a pipeline stage never landed";
    case sk::kStExpanderEmpty: return "expander: a buffer of expanded weights was never released by the MMAs that read it";
    case sk::kStMmaLdFull: return "MMA issuer: the copies of a pipeline stage never landed";
    case sk::kStMmaExFull: return "MMA issuer: the expanded weights of a stage never arrived";
    case sk::kStMmaAccEmpty: return "MMA issuer: an accumulator buffer was never released by the epilogue";
    case sk::kStEpilogueAccFull: return "epilogue: the MMAs of a scale group never completed";
    case sk::kStEpilogueScales: return "epilogue: the copy of the group scales never landed";
    case sk::kStDrain: return "producer: a copy in flight did not land while the CTA was giving up";
    case sk::kStStreamSlots: return "epilogue: a tile is shared by more CTAs than the scratch buffer has slots for";
    default: return "unknown device status";
  }
}

int sk_w2a8_query_launch(sk_w2a8_plan* plan, int64_t M, int* token_tile, int* split_k, int* ctas, int* kernel_kind) {
  if (!plan) return SK_ERR_NULL_POINTER;
  if (M <= 0) return SK_ERR_BAD_SHAPE;
  sk::LaunchChoice c;
  const int rc = sk::resolve_launch(plan, M, false, &c);
  if (rc != SK_OK) return rc;
  if (token_tile) *token_tile = c.token_tile;
  if (split_k) *split_k = c.split_k;
  if (ctas) *ctas = c.ctas;
  if (kernel_kind) *kernel_kind = c.kernel;
  return SK_OK;
}

// ---------------------------------------------------------------------------------------------- activation side
int sk_w2a8_quantize_weight(const float* w, int64_t ld_w, int64_t K, int64_t N, int group_size, uint8_t* w_packed,
                            float* scale_f32, void* scale_f16, sk_stream_t stream) {
  if (!w || !w_packed || (!scale_f32 && !scale_f16)) return SK_ERR_NULL_POINTER;
  if (K <= 0 || N <= 0 || group_size <= 0 || (group_size % 4) != 0 || (K % group_size) != 0 || ld_w < N ||
      K > (1LL << 30) || N > (1LL << 30) || K / group_size > 65535)
    return SK_ERR_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(w) & 3) || (scale_f16 && (reinterpret_cast<uintptr_t>(scale_f16) & 1)) ||
      (scale_f32 && (reinterpret_cast<uintptr_t>(scale_f32) & 3)))
    return SK_ERR_BAD_ALIGNMENT;
  const dim3 grid(static_cast<unsigned>((N + sk::kPrepThreads - 1) / sk::kPrepThreads), static_cast<unsigned>(K / group_size));
  constexpr int kPrepSmem = sk::kPrepSlab * sk::kPrepThreads * 4;     // 64 KiB
  static int prep_configured[64] = {0};
  int prep_dev = 0;
  if (cudaGetDevice(&prep_dev) != cudaSuccess) return SK_ERR_CUDA;
  if (prep_dev >= 0 && prep_dev < 64 && !prep_configured[prep_dev]) {
    if (cudaFuncSetAttribute(sk::quantize_pack_weight_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrepSmem) != cudaSuccess) {
      (void)cudaGetLastError();
      return SK_ERR_CUDA;
    }
    prep_configured[prep_dev] = 1;
  }
  sk::quantize_pack_weight_kernel<<<grid, sk::kPrepCtaThreads, kPrepSmem, static_cast<cudaStream_t>(stream)>>>(
      w, ld_w, static_cast<int>(K), static_cast<int>(N), group_size, w_packed, scale_f32, static_cast<__half*>(scale_f16));
  if (cudaGetLastError() != cudaSuccess) return SK_ERR_CUDA;
  return SK_OK;
}

int sk_quantize_activation_int8(const void* x_f16, int64_t ld_x, int64_t M, int64_t K, int8_t* x_q, int64_t ld_q,
                                float* x_scale, sk_stream_t stream) {
  if (!x_f16 || !x_q || !x_scale) return SK_ERR_NULL_POINTER;
  if (M <= 0 || K <= 0 || (K % 8) != 0 || ld_x < K || ld_q < K || M > 0x7fffffffLL) return SK_ERR_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(x_f16) & 15) || (ld_x % 8) || (reinterpret_cast<uintptr_t>(x_q) & 7) || (ld_q % 8))
    return SK_ERR_BAD_ALIGNMENT;
  auto st = static_cast<cudaStream_t>(stream);
  const __half* x = static_cast<const __half*>(x_f16);
  const dim3 grid(static_cast<unsigned>(M));
  // launched as a programmatic dependent launch: the kernel waits for its inputs itself (griddepcontrol.wait) and
  // lets the kernel behind it start its set-up early
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(sk::kActThreads, 1, 1);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const long long ldx = ld_x, ldq = ld_q;
  const int k = static_cast<int>(K);
  cudaError_t le;
  if (K <= 8 * sk::kActThreads * 2) le = cudaLaunchKernelEx(&cfg, sk::quantize_activation_kernel<2>, x, ldx, x_q, ldq, x_scale, k);
  else if (K <= 8 * sk::kActThreads * 4) le = cudaLaunchKernelEx(&cfg, sk::quantize_activation_kernel<4>, x, ldx, x_q, ldq, x_scale, k);
  else le = cudaLaunchKernelEx(&cfg, sk::quantize_activation_kernel<8>, x, ldx, x_q, ldq, x_scale, k);
  if (le != cudaSuccess) { (void)cudaGetLastError(); return SK_ERR_CUDA; }
  if (cudaGetLastError() != cudaSuccess) return SK_ERR_CUDA;
  return SK_OK;
}

int sk_silu_mul_quantize_int8(const void* gate_up_f16, int64_t ld_gu, int64_t M, int64_t I, int8_t* h_q, int64_t ld_q,
                              float* h_scale, sk_stream_t stream) {
  if (!gate_up_f16 || !h_q || !h_scale) return SK_ERR_NULL_POINTER;
  if (M <= 0 || I <= 0 || (I % 8) != 0 || ld_gu < 2 * I || ld_q < I || M > 0x7fffffffLL || I > 0x7fffffffLL)
    return SK_ERR_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(gate_up_f16) & 15) || (ld_gu % 8) || (reinterpret_cast<uintptr_t>(h_q) & 7) || (ld_q % 8))
    return SK_ERR_BAD_ALIGNMENT;
  const auto st = static_cast<cudaStream_t>(stream);
  const __half* gu = static_cast<const __half*>(gate_up_f16);
  // one pass over HBM: the row split over a cluster of 1..8 CTAs whose threads keep their fp32 values in registers
  const long long per_cta = 8LL * sk::kActThreads * sk::kClusterVecs;
  int csize = 1;
  while (csize < 8 && I > per_cta * csize) csize *= 2;
  if (I <= per_cta * csize) {
    for (int64_t m0 = 0; m0 < M; m0 += 65535) {       // gridDim.y holds at most 65535 rows per launch
      const int64_t rows = M - m0 < 65535 ? M - m0 : 65535;
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(static_cast<unsigned>(csize), static_cast<unsigned>(rows), 1);
      cfg.blockDim = dim3(sk::kActThreads, 1, 1);
      cfg.stream = st;
      cudaLaunchAttribute attr[2];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = static_cast<unsigned>(csize);
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // see sk_quantize_activation_int8
      attr[1].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 2;
      if (cudaLaunchKernelEx(&cfg, sk::silu_mul_quantize_cluster_kernel, gu + m0 * ld_gu, static_cast<long long>(ld_gu),
                             h_q + m0 * ld_q, static_cast<long long>(ld_q), h_scale + m0, static_cast<int>(I)) != cudaSuccess) {
        (void)cudaGetLastError();
        return SK_ERR_CUDA;
      }
    }
    return SK_OK;
  }
  // longer rows still: read twice and recompute (same values), full occupancy
  sk::silu_mul_quantize_twopass_kernel<<<static_cast<unsigned>(M), sk::kActThreads, 0, st>>>(
      gu, ld_gu, h_q, ld_q, h_scale, static_cast<int>(I));
  if (cudaGetLastError() != cudaSuccess) return SK_ERR_CUDA;
  return SK_OK;
}

// workspace layout of the MLP block (all offsets 256-byte aligned)
namespace {
struct MlpLayout {
  size_t x_q, x_scale, gate_up, h_q, h_scale, total;
};
inline size_t up256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }
inline MlpLayout mlp_layout(int64_t M, int64_t hidden, int64_t inter) {
  MlpLayout l;
  size_t o = 0;
  l.x_q = o;     o = up256(o + static_cast<size_t>(M) * hidden);
  l.x_scale = o; o = up256(o + static_cast<size_t>(M) * 4);
  l.gate_up = o; o = up256(o + static_cast<size_t>(M) * 2 * inter * 2);
  l.h_q = o;     o = up256(o + static_cast<size_t>(M) * inter);
  l.h_scale = o; o = up256(o + static_cast<size_t>(M) * 4);
  l.total = o;
  return l;
}
// The caller has made the plans' device current: the two side kernels launch on the current device.
int mlp_run(sk_w2a8_plan* gu, sk_w2a8_plan* down, int64_t M, const void* x, int64_t ld_x, void* out, int64_t ld_out,
            char* ws, sk_stream_t stream) {
  const int64_t hidden = gu->K, inter = down->K;
  const MlpLayout l = mlp_layout(M, hidden, inter);
  int8_t* x_q = reinterpret_cast<int8_t*>(ws + l.x_q);
  float* x_scale = reinterpret_cast<float*>(ws + l.x_scale);
  void* gate_up = ws + l.gate_up;
  int8_t* h_q = reinterpret_cast<int8_t*>(ws + l.h_q);
  float* h_scale = reinterpret_cast<float*>(ws + l.h_scale);
  int rc = sk_quantize_activation_int8(x, ld_x, M, hidden, x_q, hidden, x_scale, stream);
  if (rc == SK_OK) rc = sk_w2a8_gemm(gu, M, x_q, hidden, x_scale, gate_up, 2 * inter, stream);
  if (rc == SK_OK) rc = sk_silu_mul_quantize_int8(gate_up, 2 * inter, M, inter, h_q, inter, h_scale, stream);
  if (rc == SK_OK) rc = sk_w2a8_gemm(down, M, h_q, inter, h_scale, out, ld_out, stream);
  return rc;
}
int mlp_check(const sk_w2a8_plan* gu, const sk_w2a8_plan* down, int64_t M) {
  if (!gu || !down) return SK_ERR_NULL_POINTER;
  if (M <= 0) return SK_ERR_BAD_SHAPE;
  if (gu->N != 2 * down->K || down->N != gu->K || gu->device != down->device) return SK_ERR_BAD_SHAPE;
  if (gu->out_dtype != SK_OUT_F16) return SK_ERR_BAD_ARGUMENT;   // the SiLU kernel reads fp16
  if ((gu->K % 16) != 0 || (down->K % 16) != 0) return SK_ERR_BAD_SHAPE;
  return SK_OK;
}
}  // namespace

int64_t sk_w2a8_mlp_workspace_bytes(const sk_w2a8_plan* gate_up, const sk_w2a8_plan* down, int64_t M) {
  if (mlp_check(gate_up, down, M) != SK_OK) return 0;
  return static_cast<int64_t>(mlp_layout(M, gate_up->K, down->K).total);
}

int sk_w2a8_mlp_forward(sk_w2a8_plan* gate_up, sk_w2a8_plan* down, int64_t M, const void* x_f16, int64_t ld_x,
                        void* out, int64_t ld_out, void* workspace, int64_t workspace_bytes, sk_stream_t stream) {
  int rc = mlp_check(gate_up, down, M);
  if (rc != SK_OK) return rc;
  if (!x_f16 || !out || !workspace) return SK_ERR_NULL_POINTER;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return SK_ERR_BAD_ALIGNMENT;
  if (workspace_bytes < static_cast<int64_t>(mlp_layout(M, gate_up->K, down->K).total)) return SK_ERR_BAD_SHAPE;
  // a plan is bound to one device: run there whatever device the calling thread has current, and put that back
  const int dev = gate_up->device;
  int cur = -1;
  if (cudaGetDevice(&cur) != cudaSuccess) return sk::cuda_fail(gate_up, cudaGetLastError());
  if (cur != dev && cudaSetDevice(dev) != cudaSuccess) return sk::cuda_fail(gate_up, cudaGetLastError());
  rc = mlp_run(gate_up, down, M, x_f16, ld_x, out, ld_out, static_cast<char*>(workspace), stream);
  if (cur != dev) (void)cudaSetDevice(cur);
  return rc;
}

// ------------------------------------------------------------------------------------------------
// MLP block without any allocation: the intermediates live in a fixed array that is part of the library image.
// ------------------------------------------------------------------------------------------------
namespace {
constexpr size_t kMlpStaticBytes = 8u << 20;   // 8 MiB per GPU that loads the library, held until the process exits
static __device__ __align__(256) unsigned char g_mlp_static_scratch[kMlpStaticBytes];
std::mutex g_static_mu;
void* g_static_addr[64] = {nullptr};           // device address of the array, per device ordinal
}  // namespace

int64_t sk_w2a8_mlp_static_scratch_bytes(void) { return static_cast<int64_t>(kMlpStaticBytes); }

int sk_w2a8_mlp_forward_static(sk_w2a8_plan* gate_up, sk_w2a8_plan* down, int64_t M, const void* x_f16, int64_t ld_x,
                               void* out, int64_t ld_out, sk_stream_t stream) {
  int rc = mlp_check(gate_up, down, M);
  if (rc != SK_OK) return rc;
  if (!x_f16 || !out) return SK_ERR_NULL_POINTER;
  if (mlp_layout(M, gate_up->K, down->K).total > kMlpStaticBytes) return SK_ERR_STATIC_SCRATCH_TOO_SMALL;
  const int dev = gate_up->device;
  if (dev < 0 || dev >= 64) return SK_ERR_BAD_ARGUMENT;
  int cur = -1;
  if (cudaGetDevice(&cur) != cudaSuccess) return sk::cuda_fail(gate_up, cudaGetLastError());
  if (cur != dev && cudaSetDevice(dev) != cudaSuccess) return sk::cuda_fail(gate_up, cudaGetLastError());
  void* scratch = nullptr;
  {
    // In host code the array's name is only a handle; the address a kernel can use has to be asked for, once
    // per device and with that device current.
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!g_static_addr[dev]) {
      void* p = nullptr;
      const cudaError_t e = cudaGetSymbolAddress(&p, g_mlp_static_scratch);
      if (e != cudaSuccess || !p) {
        if (cur != dev) (void)cudaSetDevice(cur);
        return sk::cuda_fail(gate_up, e);
      }
      g_static_addr[dev] = p;
    }
    scratch = g_static_addr[dev];
  }
  rc = mlp_run(gate_up, down, M, x_f16, ld_x, out, ld_out, static_cast<char*>(scratch), stream);
  if (cur != dev) (void)cudaSetDevice(cur);
  return rc;
}

int sk_w2a8_debug_expander_image(const uint8_t* w_tiled_block, int zero_point, const int8_t* expanded_rowmajor,
                                 uint8_t* image_expander, uint8_t* image_tma, int* mismatches, int* device_status,
                                 sk_stream_t stream) {
  if (!w_tiled_block || !expanded_rowmajor || !image_expander || !image_tma || !mismatches || !device_status)
    return SK_ERR_NULL_POINTER;
  if (zero_point < 0 || zero_point > 3) return SK_ERR_BAD_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(w_tiled_block) & 15) || (reinterpret_cast<uintptr_t>(expanded_rowmajor) & 15) ||
      (reinterpret_cast<uintptr_t>(image_expander) & 15) || (reinterpret_cast<uintptr_t>(image_tma) & 15))
    return SK_ERR_BAD_ALIGNMENT;
  sk::EncodeTiledFn enc = sk::get_encode_fn();
  if (!enc) return SK_ERR_CUDA;
  CUtensorMap map;
  const cuuint64_t dims[2] = {128, 128};
  const cuuint64_t strides[1] = {128};
  const cuuint32_t box[2] = {128u, 128u};
  const cuuint32_t estr[2] = {1u, 1u};
  if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(expanded_rowmajor), dims, strides, box, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return SK_ERR_CUDA;
  const int dyn = 4096 + 2 * sk::kWxBytes + 1024;
  static int configured[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return SK_ERR_CUDA;
  if (dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(sk::expander_image_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dyn) != cudaSuccess) {
      (void)cudaGetLastError();
      return SK_ERR_CUDA;
    }
    configured[dev] = 1;
  }
  sk::expander_image_kernel<<<1, 128, dyn, static_cast<cudaStream_t>(stream)>>>(map, w_tiled_block, zero_point, image_expander,
                                                                          image_tma, mismatches, device_status);
  if (cudaGetLastError() != cudaSuccess) return SK_ERR_CUDA;
  return SK_OK;
}

int sk_w2a8_debug_stream_cut(int64_t units, int ctas, int cta, int64_t unit, int64_t* range_begin, int64_t* range_end,
                             int* owner_of_unit) {
  if (units <= 0 || ctas <= 0 || ctas > units || cta < 0 || cta >= ctas || unit < 0 || unit >= units) return SK_ERR_BAD_ARGUMENT;
  if (range_begin) *range_begin = sk::stream_range_begin(units, ctas, cta);
  if (range_end) *range_end = sk::stream_range_begin(units, ctas, cta + 1);
  if (owner_of_unit) *owner_of_unit = sk::stream_owner(units, ctas, unit);
  return SK_OK;
}

int sk_sum_row_blocks(const void* blocks, int n_blocks, int64_t block_stride, int64_t ld, int64_t rows, int64_t N,
                      void* out, int64_t ld_out, int out_dtype, sk_stream_t stream) {
  if (!blocks || !out) return SK_ERR_NULL_POINTER;
  if (n_blocks < 1 || n_blocks > 64) return SK_ERR_BAD_ARGUMENT;
  if (out_dtype != SK_OUT_F16 && out_dtype != SK_OUT_BF16) return SK_ERR_BAD_ARGUMENT;
  if (rows <= 0 || N <= 0 || (N % 8) != 0 || ld < N || ld_out < N || N > 0x7fffffffLL) return SK_ERR_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(blocks) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) || (ld % 8) || (ld_out % 8) ||
      (block_stride % 8))
    return SK_ERR_BAD_ALIGNMENT;
  const long long total = rows * (N / 8);
  const int threads = 256;
  const long long want = (total + threads - 1) / threads;
  const int grid = static_cast<int>(want < 148 * 16 ? want : 148 * 16);
  const auto st = static_cast<cudaStream_t>(stream);
  if (out_dtype == SK_OUT_BF16)
    sk::sum_row_blocks_kernel<true><<<grid, threads, 0, st>>>(static_cast<const uint16_t*>(blocks), block_stride, ld, n_blocks,
                                                             rows, static_cast<int>(N), static_cast<uint16_t*>(out), ld_out);
  else
    sk::sum_row_blocks_kernel<false><<<grid, threads, 0, st>>>(static_cast<const uint16_t*>(blocks), block_stride, ld, n_blocks,
                                                              rows, static_cast<int>(N), static_cast<uint16_t*>(out), ld_out);
  if (cudaGetLastError() != cudaSuccess) return SK_ERR_CUDA;
  return SK_OK;
}

#ifdef SK_TRACE
// Diagnostic build only: device buffer of 5 x 64 clock stamps written by CTA (0,0,0) of the next launches.
int sk_w2a8_set_trace_buffer(long long* device_buffer) {
  sk::g_trace_buffer = device_buffer;
  return SK_OK;
}
#endif

}  // extern "C"
