/*
 * sk_w2a8.h — C ABI of the B200 (sm_100a) W2A8 GEMM: 2-bit packed weights x int8 activations.
 *
 *   out[m, n] = cast( x_scale[m] * sum_g  w_scale[g, n] * fp32( sum_{k in group g} x_q[m, k] * (code[n, k] - zero_point) ) )
 *
 * Operand format (device memory, caller-owned, row-major):
 *   x_q      int8   [M, K]      leading dimension ld_x (elements = bytes), ld_x % 16 == 0, 16-byte aligned
 *   x_scale  float  [M]
 *   w_packed uint8  [N, K/4]    byte j of row n holds codes k = 4j..4j+3, k = 4j in bits 7:6
 *                               (the layout produced by the reference's matrix_packer.py:29-34)
 *   w_scale  half   [K/G, N]    per-group scales, groups along K (orientation of quantization.py:23-38)
 *   out      half | bfloat16 [M, N]  leading dimension ld_out >= N (elements)
 * Constraints: K % 32 == 0, K % G == 0, G % 32 == 0 and (G % 128 == 0 or 128 % G == 0).
 *
 * The reference has no FFI for this path; the entry points below take the place of its C++ host
 * launcher  gemm_tn(m, n, a_k, b_k, alpha, A, ldA, B, ldB, beta, C, ldC, stream)
 * (slimkernels/cute/gemm/wgmma_sm90_W2A8.cu:428-437) and keep its conventions: raw device pointers,
 * caller-owned buffers, leading dimensions in elements, output written in place.  Unlike that launcher
 * the stream argument is honoured, errors are returned (no abort, no prints) and results are stored.
 *
 * All functions return 0 (SK_OK) or a negative sk_status.  No exceptions cross this boundary.
 * Calls on one plan must be externally ordered; a plan is bound to one device.
 */
#ifndef SK_W2A8_H_
#define SK_W2A8_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct sk_w2a8_plan sk_w2a8_plan;
typedef void* sk_stream_t; /* cudaStream_t */

typedef enum sk_status {
  SK_OK = 0,
  SK_ERR_NULL_POINTER = -1,
  SK_ERR_BAD_SHAPE = -2,
  SK_ERR_BAD_ALIGNMENT = -3,
  SK_ERR_UNSUPPORTED_ARCH = -4, /* device is not compute capability 10.x */
  SK_ERR_CUDA = -5,             /* a CUDA runtime/driver call failed; see sk_w2a8_last_cuda_error */
  SK_ERR_DEVICE_TIMEOUT = -6,   /* a bounded wait inside a kernel expired; see sk_w2a8_last_device_status */
  SK_ERR_BAD_ARGUMENT = -7,
  SK_ERR_OUT_OF_MEMORY = -8,
  SK_ERR_UNAVAILABLE = -9,      /* requested kernel/option not available for this plan */
  SK_ERR_STATIC_SCRATCH_TOO_SMALL = -10 /* sk_w2a8_mlp_forward_static: the problem exceeds the fixed buffer */
} sk_status;

typedef enum sk_out_dtype { SK_OUT_F16 = 0, SK_OUT_BF16 = 1 } sk_out_dtype;

/* Layout of the weight bytes handed to sk_w2a8_plan_create. */
typedef enum sk_weight_layout {
  SK_WEIGHT_ROWMAJOR = 0, /* matrix_packer.py layout, uint8 [N, K/4]; the plan makes its own tiled copy */
  SK_WEIGHT_TILED = 1     /* output of sk_w2a8_repack; borrowed, must outlive the plan */
} sk_weight_layout;

/* Keys of sk_w2a8_set_option (testing / tuning; 0 or SK_AUTO restores the heuristic). */
typedef enum sk_option {
  SK_OPT_KERNEL = 1,      /* 0 auto, 1 general tcgen05 kernel (one CTA per tile), 2 CUDA-core checker kernel (needs
                             SK_WEIGHT_ROWMAJOR), 3 decode tcgen05 kernel that gives a CTA one feature tile or 1/2, 1/4, 1/8
                             of its K range, summed over a cluster (group size 128; used for token tiles 16 / 32, else 1 is
                             taken), 4 prefill tcgen05 kernel on pairs of CTAs (cta_group::2; group size 128, token tile 256, an
                             even number of 128-feature tiles, else 1 is taken), 5 decode tcgen05 kernel that cuts the K
                             range of the WHOLE problem into equal CTA ranges, two CTAs per SM (the default for M <= 32
                             with group size 128 and K a multiple of 256; else 3 is taken).  Partial sums of tiles that
                             two or more CTAs share meet in a scratch buffer owned by the plan, so calls on one plan
                             must not run concurrently (they must not anyway, see above). */
  SK_OPT_TOKEN_TILE = 2,  /* tokens per CTA tile: 0 auto, or 16 / 32 / 64 / 128 / 192 / 256 */
  SK_OPT_SPLIT_K = 3,     /* CTAs (one cluster) sharing the K range of one tile: 0 auto, 1, 2, 4, 8 */
  SK_OPT_TMA_STORE = 6,   /* general kernel, one CTA per tile: 0 auto (= 2), 1 vector stores by the epilogue threads, 2 one TMA
                             store per destination where alignment allows (16-byte base, pitch % 8 == 0, N % 8 == 0) */
  SK_OPT_DEPENDENT_LAUNCH = 5, /* decode kernels: 0 auto (= 2), 1 plain launch, 2 programmatic dependent launch: the
                             kernel's set-up and first weight copies overlap the tail of the previous kernel in the
                             stream; it waits for that kernel before it reads activations or writes outputs */
  SK_OPT_PERSISTENT = 4,  /* 0 auto (= 1), 1 one CTA per tile, 2 one resident set of CTAs walks all tiles (token tiles
                             128 / 256 without split-K, when there are more tiles than the GPU holds at once) */
  SK_OPT_WAIT_LIMIT_CYCLES = 7, /* SM cycles after which a wait inside a kernel gives up and the kernel returns with a
                             device status (0 = default, 1e9 cycles, about half a second; otherwise >= 1000) */
  SK_OPT_STREAM_CTAS = 9, /* kernel 5: CTAs the problem is cut into; 0 auto (two per SM, at least two K blocks each).
                             Reallocates the plan's scratch buffer: a set-up call, not for the call path. */
  SK_OPT_TEST_SKIP_COPY = 8, /* failure-path test hook, 0 = off: with value v > 0 the producer of every CTA leaves out
                             the copies of K block v - 1 of its range, so the waits for them run into the limit, the
                             kernel returns and sk_w2a8_last_device_status reports which wait gave up.  The output
                             of such a launch is undefined.  Nothing traps or faults. */
} sk_option;

/* -------- weight preparation ("Blackwell tile order") ------------------------------------------
 * The tcgen05 kernel streams weights in a tiled order: 128 output rows x 128 K-codes per 4 KiB block,
 * blocks of one 128-row tile contiguous along K, bit order inside each 32-bit word chosen so that 16
 * codes expand to 16 int8 bytes with four byte-permute look-ups.  The repack is a pure permutation of the
 * 2-bit codes (plus zero padding of N to 128 and K to 128); sk_w2a8_unrepack inverts it exactly.
 * Replaces nothing in the reference; anticipated there by its pre-tiled copy test
 * (slimkernels/cute/gemm/test_bc.cu:70-74). */
int64_t sk_w2a8_tiled_bytes(int64_t N, int64_t K);
int sk_w2a8_repack(const uint8_t* w_packed, int64_t N, int64_t K, uint8_t* w_tiled, sk_stream_t stream);
int sk_w2a8_unrepack(const uint8_t* w_tiled, int64_t N, int64_t K, uint8_t* w_packed, sk_stream_t stream);

/* -------- plan ------------------------------------------------------------------------------------
 * Binds one weight matrix to a device: validates shapes/alignment, builds the tiled weight copy (or
 * borrows one), allocates a 4-byte device status word.  Stands where gemm_tn builds its tilers, smem
 * layouts and tensor maps on every call (wgmma_sm90_W2A8.cu:448-466).  Synchronises `device` once.
 * With group size 128 the plan also makes a private copy of the scales in the order its decode kernels
 * stream them, and -- for weight matrices large enough that the balanced-split decode kernel is their default, or
 * on the first SK_OPT_KERNEL = 5 / SK_OPT_STREAM_CTAS request -- a scratch buffer for that kernel's partial sums
 * (3-20 MiB):
 * w_scale_f16 must still outlive the plan (the other kernels read it), and a change of its contents
 * after plan creation is not picked up consistently -- make a new plan instead. */
int sk_w2a8_plan_create(sk_w2a8_plan** plan, int device, int64_t N, int64_t K, int group_size,
                        int zero_point, const uint8_t* w, int w_layout, const void* w_scale_f16,
                        int out_dtype);
int sk_w2a8_plan_destroy(sk_w2a8_plan* plan);
int sk_w2a8_set_option(sk_w2a8_plan* plan, int key, int64_t value);
/* What the plan was created with (any out-pointer may be NULL). */
int sk_w2a8_plan_info(const sk_w2a8_plan* plan, int64_t* N, int64_t* K, int* group_size, int* zero_point,
                      int* out_dtype, int* device);

/* -------- the GEMM (replaces gemm_tn, wgmma_sm90_W2A8.cu:428-506) ---------------------------------
 * Stream-ordered and asynchronous; no allocation, no synchronisation. */
int sk_w2a8_gemm(sk_w2a8_plan* plan, int64_t M, const int8_t* x_q, int64_t ld_x, const float* x_scale,
                 void* out, int64_t ld_out, sk_stream_t stream);

/* The same GEMM, written to several destinations at once: the [M, N] result lands at column `col_offset` of each
 * of the n_outs (1..8) row-major buffers outs[i] of leading dimension ld_out.  outs[0] is a local buffer, the
 * others may be peer-mapped buffers of other GPUs (CUDA IPC / symmetric memory): the kernel's epilogue stores
 * every finished tile to all of them, so an N-sharded all-gather of the output overlaps the GEMM.  Where every
 * destination is 16-byte aligned, ld_out % 8 == 0 and N % 8 == 0 a tile leaves as one TMA store per destination
 * (stores only: nothing is ever loaded from a peer, and no multicast is used); otherwise the epilogue threads
 * store 16-byte vectors or single elements.  The caller synchronises the ranks afterwards.  No counterpart in the
 * reference (single-GPU only). */
int sk_w2a8_gemm_scatter(sk_w2a8_plan* plan, int64_t M, const int8_t* x_q, int64_t ld_x, const float* x_scale,
                         void* const* outs, int n_outs, int64_t ld_out, int64_t col_offset, sk_stream_t stream);

/* The same GEMM with its token rows dealt out: rows [d * rows_per_dest, (d + 1) * rows_per_dest) of the [M, N]
 * result go to destination outs[d] ONLY (n_outs = 1..8, M == n_outs * rows_per_dest), where they land at rows
 * dst_row0 .. dst_row0 + rows_per_dest - 1 of a row-major buffer of leading dimension ld_out.  This is the
 * scatter half of a reduce-scatter: with the weight split along K over R ranks, rank r calls it with
 * outs[d] = rank d's [R * rows_per_dest, N] buffer (peer-mapped for d != r) and dst_row0 = r * rows_per_dest, so that
 * after a barrier rank d holds the R partial sums of its rows, block r from rank r, and adds them in rank order.
 * Stores only (TMA stores of whole tiles where alignment allows, as for sk_w2a8_gemm_scatter); nothing is loaded
 * from a peer.  rows_per_dest must be a multiple of the token tile the plan uses for M (256 for M > 128), and the
 * launch must be the general kernel's: SK_ERR_UNAVAILABLE otherwise.  No counterpart in the reference. */
int sk_w2a8_gemm_rowscatter(sk_w2a8_plan* plan, int64_t M, const int8_t* x_q, int64_t ld_x, const float* x_scale,
                            void* const* outs, int n_outs, int64_t rows_per_dest, int64_t dst_row0, int64_t ld_out,
                            sk_stream_t stream);

/* The add half of a reduce-scatter of K-sharded partial sums: out[r, n] = round( sum_b fp32(blocks[b][r][n]) ), the
 * n_blocks (1..64) row blocks [rows, N] of 16-bit floats (out_dtype says which) added in fp32 in block order and
 * rounded once.  Block b starts block_stride elements after block b - 1; row pitches ld / ld_out; N % 8 == 0,
 * 16-byte aligned pointers and pitches.  One pass over the data.  No counterpart in the reference. */
int sk_sum_row_blocks(const void* blocks, int n_blocks, int64_t block_stride, int64_t ld, int64_t rows, int64_t N,
                      void* out, int64_t ld_out, int out_dtype, sk_stream_t stream);

/* Test aid.  Expands ONE tiled 128 x 128 weight block (4096 bytes, device) the way the general kernel's expander
 * threads do -- 2-bit codes -> int8 (code - zero_point), stored in the 128-byte-swizzled K-major shared-memory
 * layout -- and, next to it, lets the TMA load the same block given pre-expanded (int8 [128 rows][128 codes],
 * row-major, device) through a tensor map with 128-byte swizzle.  Both 16 KiB shared-memory images are copied out
 * (image_expander, image_tma) and *mismatches (zero it first) receives the number of bytes that differ; *device_status
 * (zero it first) is set if the bounded wait for the TMA expired.  Follows the staging check of the reference's
 * test_tma.cu (slimkernels/cute/gemm/test_tma.cu), which prints what a TMA load left in shared memory. */
int sk_w2a8_debug_expander_image(const uint8_t* w_tiled_block, int zero_point, const int8_t* expanded_rowmajor,
                                 uint8_t* image_expander, uint8_t* image_tma, int* mismatches, int* device_status,
                                 sk_stream_t stream);

/* Test aid, host only (no device is touched): the cut of the balanced-split decode kernel.  With `units` half stages
 * dealt to `ctas` CTAs, CTA `cta` owns [*range_begin, *range_end); *owner_of_unit is the CTA whose range holds `unit`.
 * The kernel and the host size their slots with these two formulas; a test checks that they agree for every unit. */
int sk_w2a8_debug_stream_cut(int64_t units, int ctas, int cta, int64_t unit, int64_t* range_begin, int64_t* range_end,
                             int* owner_of_unit);

/* Same contraction, but stores the exact per-group integer partial sums
 * partials[g, m, n] (int32, [K/G, M, N] contiguous) instead of the scaled output. */
int sk_w2a8_gemm_debug_partials(sk_w2a8_plan* plan, int64_t M, const int8_t* x_q, int64_t ld_x,
                                int32_t* partials, sk_stream_t stream);

/* -------- weight preparation on the GPU ---------------------------------------------------------------
 * Replaces, for a float32 weight, the host composition  quantize_to_uint2 (quantization.py:3-53)  then
 * pack_matrix on the transposed codes (matrix_packer.py:3-36), bit for bit (same IEEE float32 operations: the
 * 1e-9 floor, true division, round half to even, zero point 1).
 *   w         float  [K, ld_w]   W[k, n], k = in-feature (groups of group_size rows along K), n = out-feature
 *   w_packed  uint8  [N, K/4]    out, matrix_packer layout (what sk_w2a8_plan_create takes)
 *   scale_f32 float  [K/G, N]    out or NULL: the scales as quantize_to_uint2 returns them
 *   scale_f16 half   [K/G, N]    out or NULL: rounded to nearest even, what the GEMM consumes
 * group_size % 4 == 0, K % group_size == 0, ld_w >= N.  Inputs must be finite. */
int sk_w2a8_quantize_weight(const float* w, int64_t ld_w, int64_t K, int64_t N, int group_size, uint8_t* w_packed,
                            float* scale_f32, void* scale_f16, sk_stream_t stream);

/* -------- activation side of the Llama MLP block -----------------------------------------------------
 * The reference has no activation quantiser (its prototype is fed ready-made e4m3 tensors,
 * wgmma_sm90_W2A8.cu:541-552).  Definition used here, per token row:
 *   s = max|x| / 127 (1.0 for an all-zero row),  q = clamp(round_half_even(x / s), -127, 127).
 * x fp16 [M, ld_x] -> x_q int8 [M, ld_q], x_scale fp32 [M].  K % 8 == 0, rows 16-byte aligned. */
int sk_quantize_activation_int8(const void* x_f16, int64_t ld_x, int64_t M, int64_t K, int8_t* x_q, int64_t ld_q,
                                float* x_scale, sk_stream_t stream);
/* gate_up fp16 [M, ld_gu] (gate = columns [0, I), up = [I, 2I)) -> h = SiLU(gate) * up in fp32, quantised as
 * above to h_q int8 [M, ld_q], h_scale fp32 [M].  I % 8 == 0. */
int sk_silu_mul_quantize_int8(const void* gate_up_f16, int64_t ld_gu, int64_t M, int64_t I, int8_t* h_q,
                              int64_t ld_q, float* h_scale, sk_stream_t stream);
/* The whole block: quantise x, W2A8 GEMM with the fused gate+up weight ([2I, hidden] packed, gate rows first),
 * SiLU*up + re-quantise, W2A8 GEMM with the down weight ([hidden, I]).  The intermediates live in a
 * caller-provided device workspace of sk_w2a8_mlp_workspace_bytes(...) bytes (256-byte aligned); nothing is
 * allocated.  gate_up's plan must produce fp16.  Four launches on `stream`, no synchronisation. */
int64_t sk_w2a8_mlp_workspace_bytes(const sk_w2a8_plan* gate_up, const sk_w2a8_plan* down, int64_t M);
int sk_w2a8_mlp_forward(sk_w2a8_plan* gate_up, sk_w2a8_plan* down, int64_t M, const void* x_f16, int64_t ld_x,
                        void* out, int64_t ld_out, void* workspace, int64_t workspace_bytes, sk_stream_t stream);

/* The MLP block for hosts that must not allocate device memory while serving.  It has no counterpart in the
 * reference.  Some embedders hand the GPU's memory to another owner at start-up (an inference server's arena, a
 * game or robotics runtime with a fixed budget) or run where cudaMalloc is forbidden because it synchronises the
 * device and can fail late; they can neither allocate the workspace sk_w2a8_mlp_forward asks for nor let a
 * framework do it.  This entry point performs the same four launches with the intermediates in an 8 MiB array
 * that is part of the library image (every GPU that loads the library holds those 8 MiB until the process
 * exits).  It calls no cudaMalloc / cudaFree and no allocating library routine; inputs and outputs are still the
 * caller's.  Limits and rules:
 *   - the intermediates must fit: M*hidden + 5*M*inter + 8*M bytes (each part rounded up to 256) <=
 *     sk_w2a8_mlp_static_scratch_bytes(); e.g. Llama-2-7B (hidden 4096, inter 11008) up to M = 141 tokens.
 *     Larger problems are refused with SK_ERR_STATIC_SCRATCH_TOO_SMALL and nothing is launched;
 *   - the first call on a device looks up the array's device address (cudaGetSymbolAddress, with that device made
 *     current); make that first call outside any stream capture;
 *   - all calls on one GPU share the one array, which keeps whatever the previous call left in it (every byte a
 *     call reads it has written first, so nothing needs clearing); two calls that overlap on the GPU — different
 *     streams, or different threads — race on it.  Keep such calls on one stream or order them yourself. */
int64_t sk_w2a8_mlp_static_scratch_bytes(void);
int sk_w2a8_mlp_forward_static(sk_w2a8_plan* gate_up, sk_w2a8_plan* down, int64_t M, const void* x_f16,
                               int64_t ld_x, void* out, int64_t ld_out, sk_stream_t stream);

/* -------- diagnostics -----------------------------------------------------------------------------*/
/* Synchronously reads (and clears) the plan's device status word: 0, or a code naming the wait that
 * expired inside the kernel (role * 16 + barrier kind).  Non-zero maps to SK_ERR_DEVICE_TIMEOUT. */
int sk_w2a8_last_device_status(sk_w2a8_plan* plan, int* device_status);
/* Names the role and the wait behind a device status code (static string). */
const char* sk_device_status_string(int device_status);
int sk_w2a8_last_cuda_error(const sk_w2a8_plan* plan);
/* Describes the launch the plan would make for M tokens: token tile, split-K factor, CTAs, kernel kind. */
int sk_w2a8_query_launch(sk_w2a8_plan* plan, int64_t M, int* token_tile, int* split_k, int* ctas,
                         int* kernel_kind);
/* Measurement aid (decode-sized M only, else SK_ERR_UNAVAILABLE): launches an EMPTY kernel with the grid, cluster,
 * block size, shared memory and launch attributes sk_w2a8_gemm would use for M tokens, doing only the fixed per-CTA
 * work (barrier set-up, tensor-memory allocation and release, the barriers).  Timed as a chain in a CUDA graph it gives
 * the per-launch floor of this launch geometry, against which the GEMM's time is to be read.  No counterpart in the
 * reference. */
int sk_w2a8_launch_floor_probe(sk_w2a8_plan* plan, int64_t M, sk_stream_t stream);
const char* sk_status_string(int status);
int sk_w2a8_version(void);

#ifdef __cplusplus
}
#endif
#endif /* SK_W2A8_H_ */
