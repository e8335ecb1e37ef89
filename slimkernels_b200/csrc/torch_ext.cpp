// PyTorch C++ extension: marshals tensors into the C ABI of include/sk_w2a8.h.  No kernels live here.
// Registers the ops of namespace `slimkernels` used by slimkernels_b200/torch/ops.py.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/types.h>

#include <mutex>
#include <vector>

#include "../../include/sk_w2a8.h"

namespace {

void check(int rc, const char* what) {
  TORCH_CHECK(rc == SK_OK, "slimkernels::", what, " failed: ", sk_status_string(rc), " (", rc, ")");
}

sk_w2a8_plan* as_plan(int64_t handle) {
  TORCH_CHECK(handle != 0, "slimkernels: null plan handle");
  return reinterpret_cast<sk_w2a8_plan*>(static_cast<intptr_t>(handle));
}

int64_t plan_create(const at::Tensor& w, const at::Tensor& w_scale, int64_t N, int64_t K, int64_t group_size,
                    int64_t zero_point, bool bf16_out, bool tiled) {
  TORCH_CHECK(w.is_cuda() && w_scale.is_cuda(), "slimkernels::w2a8_plan_create: weights must be CUDA tensors");
  TORCH_CHECK(w.scalar_type() == at::kByte && w.is_contiguous(), "w must be contiguous uint8");
  TORCH_CHECK(w_scale.scalar_type() == at::kHalf && w_scale.is_contiguous(), "w_scale must be contiguous float16");
  TORCH_CHECK(group_size > 0 && K % group_size == 0, "K must be a multiple of group_size");
  TORCH_CHECK(w_scale.dim() == 2 && w_scale.size(0) == K / group_size && w_scale.size(1) == N,
              "w_scale must have shape [K/group_size, N]");
  if (tiled) {
    TORCH_CHECK(w.numel() == sk_w2a8_tiled_bytes(N, K), "tiled weight has the wrong size");
  } else {
    TORCH_CHECK(w.dim() == 2 && w.size(0) == N && w.size(1) * 4 == K, "w_packed must have shape [N, K/4]");
  }
  c10::cuda::CUDAGuard guard(w.device());
  sk_w2a8_plan* plan = nullptr;
  check(sk_w2a8_plan_create(&plan, w.get_device(), N, K, static_cast<int>(group_size), static_cast<int>(zero_point),
                            w.data_ptr<uint8_t>(), tiled ? SK_WEIGHT_TILED : SK_WEIGHT_ROWMAJOR, w_scale.data_ptr(),
                            bf16_out ? SK_OUT_BF16 : SK_OUT_F16),
        "w2a8_plan_create");
  return static_cast<int64_t>(reinterpret_cast<intptr_t>(plan));
}

void plan_destroy(int64_t handle) { check(sk_w2a8_plan_destroy(as_plan(handle)), "w2a8_plan_destroy"); }

void plan_set_option(int64_t handle, int64_t key, int64_t value) {
  check(sk_w2a8_set_option(as_plan(handle), static_cast<int>(key), value), "w2a8_set_option");
}

void check_x(const at::Tensor& x_q, int64_t K) {
  TORCH_CHECK(x_q.is_cuda() && x_q.scalar_type() == at::kChar && x_q.dim() == 2, "x_q must be a 2-D CUDA int8 tensor");
  TORCH_CHECK(x_q.size(1) == K && x_q.stride(1) == 1, "x_q must be [M, K] with unit inner stride");
}

// out may be a column slice of a wider [M, N_total] buffer (stride(0) >= N): used for N-sharded execution.
void gemm_out(int64_t handle, const at::Tensor& x_q, const at::Tensor& x_scale, at::Tensor& out, int64_t K) {
  check_x(x_q, K);
  const int64_t M = x_q.size(0);
  TORCH_CHECK(x_scale.is_cuda() && x_scale.scalar_type() == at::kFloat && x_scale.is_contiguous() &&
                  x_scale.numel() == M, "x_scale must be contiguous float32 [M]");
  TORCH_CHECK(out.is_cuda() && out.dim() == 2 && out.size(0) == M && out.stride(1) == 1,
              "out must be [M, N] with unit inner stride");
  TORCH_CHECK(out.scalar_type() == at::kHalf || out.scalar_type() == at::kBFloat16, "out must be float16 or bfloat16");
  int64_t plan_n = 0, plan_k = 0;
  int plan_dtype = 0, plan_dev = 0;
  check(sk_w2a8_plan_info(as_plan(handle), &plan_n, &plan_k, nullptr, nullptr, &plan_dtype, &plan_dev), "w2a8_plan_info");
  TORCH_CHECK(out.size(1) == plan_n && K == plan_k, "out must have N = ", plan_n, " columns and x_q K = ", plan_k);
  TORCH_CHECK((out.scalar_type() == at::kBFloat16) == (plan_dtype == SK_OUT_BF16),
              "out has dtype ", out.scalar_type(), " but the plan produces ", plan_dtype == SK_OUT_BF16 ? "bfloat16" : "float16");
  TORCH_CHECK(out.get_device() == plan_dev && x_q.get_device() == plan_dev, "tensors must live on the plan's device ", plan_dev);
  if (M == 0) return;
  c10::cuda::CUDAGuard guard(x_q.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  check(sk_w2a8_gemm(as_plan(handle), M, x_q.data_ptr<int8_t>(), x_q.stride(0), x_scale.data_ptr<float>(),
                     out.data_ptr(), out.stride(0), stream.stream()),
        "w2a8_gemm");
}

// outs: raw device pointers (this rank's buffer first, then peer-mapped buffers) of [M, ld_out] row-major buffers
void gemm_scatter(int64_t handle, const at::Tensor& x_q, const at::Tensor& x_scale, std::vector<int64_t> out_ptrs,
                  int64_t ld_out, int64_t col_offset, int64_t K) {
  check_x(x_q, K);
  const int64_t M = x_q.size(0);
  TORCH_CHECK(x_scale.is_cuda() && x_scale.scalar_type() == at::kFloat && x_scale.is_contiguous() &&
                  x_scale.numel() == M, "x_scale must be contiguous float32 [M]");
  TORCH_CHECK(!out_ptrs.empty() && out_ptrs.size() <= 8, "1..8 destinations");
  if (M == 0) return;
  std::vector<void*> ptrs;
  for (int64_t v : out_ptrs) ptrs.push_back(reinterpret_cast<void*>(static_cast<intptr_t>(v)));
  c10::cuda::CUDAGuard guard(x_q.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  check(sk_w2a8_gemm_scatter(as_plan(handle), M, x_q.data_ptr<int8_t>(), x_q.stride(0), x_scale.data_ptr<float>(),
                             ptrs.data(), static_cast<int>(ptrs.size()), ld_out, col_offset, stream.stream()),
        "w2a8_gemm_scatter");
}

// outs[d]: raw device pointer of rank d's [n_outs * rows_per_dest, ld_out] buffer (peer-mapped unless it is this rank's)
void gemm_rowscatter(int64_t handle, const at::Tensor& x_q, const at::Tensor& x_scale, std::vector<int64_t> out_ptrs,
                     int64_t rows_per_dest, int64_t dst_row0, int64_t ld_out, int64_t K) {
  check_x(x_q, K);
  const int64_t M = x_q.size(0);
  TORCH_CHECK(x_scale.is_cuda() && x_scale.scalar_type() == at::kFloat && x_scale.is_contiguous() &&
                  x_scale.numel() == M, "x_scale must be contiguous float32 [M]");
  TORCH_CHECK(!out_ptrs.empty() && out_ptrs.size() <= 8, "1..8 destinations");
  TORCH_CHECK(M > 0, "no tokens");
  std::vector<void*> ptrs;
  for (int64_t v : out_ptrs) ptrs.push_back(reinterpret_cast<void*>(static_cast<intptr_t>(v)));
  c10::cuda::CUDAGuard guard(x_q.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  check(sk_w2a8_gemm_rowscatter(as_plan(handle), M, x_q.data_ptr<int8_t>(), x_q.stride(0), x_scale.data_ptr<float>(),
                                ptrs.data(), static_cast<int>(ptrs.size()), rows_per_dest, dst_row0, ld_out,
                                stream.stream()),
        "w2a8_gemm_rowscatter");
}

// blocks [B, rows, N] (half or bfloat16, contiguous) -> [rows, N]: fp32 sum over B in index order, rounded once
at::Tensor sum_row_blocks(const at::Tensor& blocks) {
  TORCH_CHECK(blocks.is_cuda() && blocks.dim() == 3 && blocks.is_contiguous(), "blocks must be a contiguous CUDA tensor [B, rows, N]");
  TORCH_CHECK(blocks.scalar_type() == at::kHalf || blocks.scalar_type() == at::kBFloat16, "blocks must be float16 or bfloat16");
  const int64_t B = blocks.size(0), rows = blocks.size(1), N = blocks.size(2);
  at::Tensor out = at::empty({rows, N}, blocks.options());
  if (rows == 0 || N == 0) return out;
  c10::cuda::CUDAGuard guard(blocks.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  check(sk_sum_row_blocks(blocks.data_ptr(), static_cast<int>(B), rows * N, N, rows, N, out.data_ptr(), N,
                          blocks.scalar_type() == at::kBFloat16 ? SK_OUT_BF16 : SK_OUT_F16, stream.stream()),
        "sum_row_blocks");
  return out;
}

at::Tensor gemm(int64_t handle, const at::Tensor& x_q, const at::Tensor& x_scale, int64_t N, int64_t K, bool bf16_out) {
  at::Tensor out = at::empty({x_q.size(0), N}, x_q.options().dtype(bf16_out ? at::kBFloat16 : at::kHalf));
  gemm_out(handle, x_q, x_scale, out, K);
  return out;
}

at::Tensor partials(int64_t handle, const at::Tensor& x_q, int64_t N, int64_t K, int64_t group_size) {
  check_x(x_q, K);
  const int64_t M = x_q.size(0);
  at::Tensor out = at::empty({K / group_size, M, N}, x_q.options().dtype(at::kInt));
  if (M == 0) return out;
  c10::cuda::CUDAGuard guard(x_q.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  check(sk_w2a8_gemm_debug_partials(as_plan(handle), M, x_q.data_ptr<int8_t>(), x_q.stride(0), out.data_ptr<int32_t>(),
                                    stream.stream()),
        "w2a8_gemm_debug_partials");
  return out;
}

// float32 W[K, N] -> (w_packed uint8 [N, K/4], w_scale float16 [K/G, N], scales float32 [K/G, N])
std::tuple<at::Tensor, at::Tensor, at::Tensor> quantize_weight(const at::Tensor& w_kn, int64_t group_size) {
  TORCH_CHECK(w_kn.is_cuda() && w_kn.scalar_type() == at::kFloat && w_kn.dim() == 2 && w_kn.stride(1) == 1,
              "w must be a 2-D CUDA float32 tensor [K, N] with unit inner stride");
  const int64_t K = w_kn.size(0), N = w_kn.size(1);
  TORCH_CHECK(group_size > 0 && group_size % 4 == 0 && K % group_size == 0, "K must be a multiple of group_size (a multiple of 4)");
  at::Tensor packed = at::empty({N, K / 4}, w_kn.options().dtype(at::kByte));
  at::Tensor s16 = at::empty({K / group_size, N}, w_kn.options().dtype(at::kHalf));
  at::Tensor s32 = at::empty({K / group_size, N}, w_kn.options().dtype(at::kFloat));
  if (K == 0 || N == 0) return {packed, s16, s32};
  c10::cuda::CUDAGuard guard(w_kn.device());
  check(sk_w2a8_quantize_weight(w_kn.data_ptr<float>(), w_kn.stride(0), K, N, static_cast<int>(group_size),
                                packed.data_ptr<uint8_t>(), s32.data_ptr<float>(), s16.data_ptr(),
                                at::cuda::getCurrentCUDAStream().stream()),
        "w2a8_quantize_weight");
  return {packed, s16, s32};
}

std::tuple<at::Tensor, at::Tensor> quantize_activation(const at::Tensor& x) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kHalf && x.dim() == 2 && x.stride(1) == 1,
              "x must be a 2-D CUDA float16 tensor with unit inner stride");
  const int64_t M = x.size(0), K = x.size(1);
  at::Tensor q = at::empty({M, K}, x.options().dtype(at::kChar));
  at::Tensor s = at::empty({M}, x.options().dtype(at::kFloat));
  if (M == 0) return {q, s};
  c10::cuda::CUDAGuard guard(x.device());
  check(sk_quantize_activation_int8(x.data_ptr(), x.stride(0), M, K, q.data_ptr<int8_t>(), K, s.data_ptr<float>(),
                                    at::cuda::getCurrentCUDAStream().stream()),
        "quantize_activation_int8");
  return {q, s};
}

std::tuple<at::Tensor, at::Tensor> silu_mul_quantize(const at::Tensor& gate_up) {
  TORCH_CHECK(gate_up.is_cuda() && gate_up.scalar_type() == at::kHalf && gate_up.dim() == 2 && gate_up.stride(1) == 1 &&
                  gate_up.size(1) % 2 == 0, "gate_up must be a 2-D CUDA float16 tensor [M, 2I]");
  const int64_t M = gate_up.size(0), I = gate_up.size(1) / 2;
  at::Tensor q = at::empty({M, I}, gate_up.options().dtype(at::kChar));
  at::Tensor s = at::empty({M}, gate_up.options().dtype(at::kFloat));
  if (M == 0) return {q, s};
  c10::cuda::CUDAGuard guard(gate_up.device());
  check(sk_silu_mul_quantize_int8(gate_up.data_ptr(), gate_up.stride(0), M, I, q.data_ptr<int8_t>(), I,
                                  s.data_ptr<float>(), at::cuda::getCurrentCUDAStream().stream()),
        "silu_mul_quantize_int8");
  return {q, s};
}

at::Tensor mlp_forward(int64_t gate_up_plan, int64_t down_plan, const at::Tensor& x, int64_t hidden_out, bool bf16_out) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kHalf && x.dim() == 2 && x.stride(1) == 1,
              "x must be a 2-D CUDA float16 tensor with unit inner stride");
  const int64_t M = x.size(0);
  at::Tensor out = at::empty({M, hidden_out}, x.options().dtype(bf16_out ? at::kBFloat16 : at::kHalf));
  if (M == 0) return out;
  const int64_t bytes = sk_w2a8_mlp_workspace_bytes(as_plan(gate_up_plan), as_plan(down_plan), M);
  TORCH_CHECK(bytes > 0, "slimkernels::w2a8_mlp_forward: the two plans do not form an MLP block");
  at::Tensor ws = at::empty({bytes}, x.options().dtype(at::kByte));     // caching allocator: 512-byte aligned
  c10::cuda::CUDAGuard guard(x.device());
  check(sk_w2a8_mlp_forward(as_plan(gate_up_plan), as_plan(down_plan), M, x.data_ptr(), x.stride(0), out.data_ptr(),
                            out.stride(0), ws.data_ptr(), bytes, at::cuda::getCurrentCUDAStream().stream()),
        "w2a8_mlp_forward");
  return out;
}

// [token tile, split-K, CTAs, kernel kind] of the launch the plan makes for M tokens
std::vector<int64_t> query_launch(int64_t handle, int64_t M) {
  int t = 0, sp = 0, c = 0, k = 0;
  check(sk_w2a8_query_launch(as_plan(handle), M, &t, &sp, &c, &k), "w2a8_query_launch");
  return {t, sp, c, k};
}

void launch_floor_probe(int64_t handle, const at::Tensor& on_device_of, int64_t M) {
  c10::cuda::CUDAGuard guard(on_device_of.device());
  check(sk_w2a8_launch_floor_probe(as_plan(handle), M, at::cuda::getCurrentCUDAStream().stream()), "w2a8_launch_floor_probe");
}

int64_t device_status(int64_t handle) {
  int v = 0;
  int rc = sk_w2a8_last_device_status(as_plan(handle), &v);
  TORCH_CHECK(rc == SK_OK || rc == SK_ERR_DEVICE_TIMEOUT, "slimkernels::w2a8_device_status failed: ", sk_status_string(rc));
  return v;
}

at::Tensor repack(const at::Tensor& w_packed) {
  TORCH_CHECK(w_packed.is_cuda() && w_packed.scalar_type() == at::kByte && w_packed.is_contiguous() && w_packed.dim() == 2,
              "w_packed must be a contiguous 2-D CUDA uint8 tensor");
  const int64_t N = w_packed.size(0), K = w_packed.size(1) * 4;
  at::Tensor out = at::empty({sk_w2a8_tiled_bytes(N, K)}, w_packed.options());
  c10::cuda::CUDAGuard guard(w_packed.device());
  check(sk_w2a8_repack(w_packed.data_ptr<uint8_t>(), N, K, out.data_ptr<uint8_t>(), at::cuda::getCurrentCUDAStream().stream()),
        "w2a8_repack");
  return out;
}

at::Tensor unrepack(const at::Tensor& w_tiled, int64_t N, int64_t K) {
  TORCH_CHECK(w_tiled.is_cuda() && w_tiled.scalar_type() == at::kByte && w_tiled.is_contiguous() &&
                  w_tiled.numel() == sk_w2a8_tiled_bytes(N, K), "w_tiled has the wrong type or size");
  at::Tensor out = at::empty({N, K / 4}, w_tiled.options());
  c10::cuda::CUDAGuard guard(w_tiled.device());
  check(sk_w2a8_unrepack(w_tiled.data_ptr<uint8_t>(), N, K, out.data_ptr<uint8_t>(), at::cuda::getCurrentCUDAStream().stream()),
        "w2a8_unrepack");
  return out;
}

// ------------------------------------------------------------------------------------------------
// The functional op.  Call shape of the reference's notebook wrapper  wint2_gemm(activation, weight, scale) -> out
// (triton.ipynb:235-270): operands in, a fresh [M, N] tensor out, on the current stream.  The plan behind a weight
// (its tiled copy) is made on first use and kept in a small cache that holds the weight tensors WEAKLY: an entry
// dies with its tensors, and is rebuilt if they were written in place.
// ------------------------------------------------------------------------------------------------
struct CachedPlan {
  c10::weak_intrusive_ptr<c10::TensorImpl> w, s;
  const void* w_ptr;
  const void* s_ptr;
  int64_t w_version, s_version;
  int64_t group_size, zero_point;
  bool bf16;
  sk_w2a8_plan* plan;
};
std::mutex g_cache_mu;
std::vector<CachedPlan> g_cache;
constexpr size_t kMaxCachedPlans = 512;

sk_w2a8_plan* cached_plan(const at::Tensor& w_packed, const at::Tensor& w_scale, int64_t group_size, int64_t zero_point,
                          bool bf16) {
  TORCH_CHECK(w_packed.is_cuda() && w_packed.scalar_type() == at::kByte && w_packed.is_contiguous() && w_packed.dim() == 2,
              "w_packed must be a contiguous 2-D CUDA uint8 tensor [N, K/4]");
  const int64_t N = w_packed.size(0), K = w_packed.size(1) * 4;
  std::lock_guard<std::mutex> lock(g_cache_mu);
  sk_w2a8_plan* hit = nullptr;
  for (size_t i = 0; i < g_cache.size();) {
    CachedPlan& e = g_cache[i];
    const bool dead = e.w.expired() || e.s.expired();
    const bool same = !dead && e.w_ptr == w_packed.data_ptr() && e.s_ptr == w_scale.data_ptr() &&
                      e.w.lock().get() == w_packed.unsafeGetTensorImpl() && e.s.lock().get() == w_scale.unsafeGetTensorImpl() &&
                      e.group_size == group_size && e.zero_point == zero_point && e.bf16 == bf16;
    const bool stale = same && (e.w_version != w_packed._version() || e.s_version != w_scale._version());
    if (dead || stale) {
      sk_w2a8_plan_destroy(e.plan);
      g_cache[i] = g_cache.back();
      g_cache.pop_back();
      continue;
    }
    if (same) hit = e.plan;
    ++i;
  }
  if (hit) return hit;
  if (g_cache.size() >= kMaxCachedPlans) {      // oldest first
    sk_w2a8_plan_destroy(g_cache.front().plan);
    g_cache.erase(g_cache.begin());
  }
  const int64_t handle = plan_create(w_packed, w_scale, N, K, group_size, zero_point, bf16, /*tiled=*/false);
  CachedPlan e{c10::weak_intrusive_ptr<c10::TensorImpl>(w_packed.getIntrusivePtr()),
               c10::weak_intrusive_ptr<c10::TensorImpl>(w_scale.getIntrusivePtr()),
               w_packed.data_ptr(), w_scale.data_ptr(), w_packed._version(), w_scale._version(),
               group_size, zero_point, bf16, as_plan(handle)};
  g_cache.push_back(e);
  return e.plan;
}

at::Tensor w2a8_gemm_op(const at::Tensor& x_q, const at::Tensor& x_scale, const at::Tensor& w_packed,
                        const at::Tensor& w_scale, int64_t group_size, int64_t zero_point, at::ScalarType out_dtype) {
  TORCH_CHECK(out_dtype == at::kHalf || out_dtype == at::kBFloat16, "out_dtype must be float16 or bfloat16");
  const bool bf16 = out_dtype == at::kBFloat16;
  sk_w2a8_plan* plan = cached_plan(w_packed, w_scale, group_size, zero_point, bf16);
  return gemm(static_cast<int64_t>(reinterpret_cast<intptr_t>(plan)), x_q, x_scale, w_packed.size(0), w_packed.size(1) * 4, bf16);
}

at::Tensor w2a8_partials_op(const at::Tensor& x_q, const at::Tensor& w_packed, const at::Tensor& w_scale,
                            int64_t group_size, int64_t zero_point) {
  sk_w2a8_plan* plan = cached_plan(w_packed, w_scale, group_size, zero_point, false);
  return partials(static_cast<int64_t>(reinterpret_cast<intptr_t>(plan)), x_q, w_packed.size(0), w_packed.size(1) * 4, group_size);
}

int64_t cached_plan_count() {
  std::lock_guard<std::mutex> lock(g_cache_mu);
  size_t live = 0;
  for (const auto& e : g_cache) live += !(e.w.expired() || e.s.expired());
  return static_cast<int64_t>(live);
}

}  // namespace

TORCH_LIBRARY(slimkernels, m) {
  m.def("w2a8_gemm(Tensor x_q, Tensor x_scale, Tensor w_packed, Tensor w_scale, int group_size=128, int zero_point=1, ScalarType out_dtype=float16) -> Tensor", &w2a8_gemm_op);
  m.def("w2a8_partials(Tensor x_q, Tensor w_packed, Tensor w_scale, int group_size=128, int zero_point=1) -> Tensor", &w2a8_partials_op);
  m.def("w2a8_cached_plan_count() -> int", &cached_plan_count);
  m.def("w2a8_plan_create(Tensor w, Tensor w_scale, int N, int K, int group_size, int zero_point, bool bf16_out, bool tiled) -> int", &plan_create);
  m.def("w2a8_plan_destroy(int plan) -> ()", &plan_destroy);
  m.def("w2a8_plan_set_option(int plan, int key, int value) -> ()", &plan_set_option);
  m.def("w2a8_plan_gemm(int plan, Tensor x_q, Tensor x_scale, int N, int K, bool bf16_out) -> Tensor", &gemm);
  m.def("w2a8_plan_gemm_out(int plan, Tensor x_q, Tensor x_scale, Tensor(a!) out, int K) -> ()", &gemm_out);
  m.def("w2a8_plan_gemm_scatter(int plan, Tensor x_q, Tensor x_scale, int[] out_ptrs, int ld_out, int col_offset, int K) -> ()", &gemm_scatter);
  m.def("w2a8_plan_gemm_rowscatter(int plan, Tensor x_q, Tensor x_scale, int[] out_ptrs, int rows_per_dest, int dst_row0, int ld_out, int K) -> ()", &gemm_rowscatter);
  m.def("sum_row_blocks(Tensor blocks) -> Tensor", &sum_row_blocks);
  m.def("w2a8_plan_partials(int plan, Tensor x_q, int N, int K, int group_size) -> Tensor", &partials);
  m.def("w2a8_plan_device_status(int plan) -> int", &device_status);
  m.def("w2a8_plan_query_launch(int plan, int M) -> int[]", &query_launch);
  m.def("w2a8_plan_launch_floor_probe(int plan, Tensor on_device_of, int M) -> ()", &launch_floor_probe);
  m.def("quantize_activation_int8(Tensor x) -> (Tensor, Tensor)", &quantize_activation);
  m.def("w2a8_quantize_weight(Tensor w_kn, int group_size) -> (Tensor, Tensor, Tensor)", &quantize_weight);
  m.def("silu_mul_quantize_int8(Tensor gate_up) -> (Tensor, Tensor)", &silu_mul_quantize);
  m.def("w2a8_mlp_forward(int gate_up_plan, int down_plan, Tensor x, int hidden_out, bool bf16_out) -> Tensor", &mlp_forward);
  m.def("w2a8_repack(Tensor w_packed) -> Tensor", &repack);
  m.def("w2a8_unrepack(Tensor w_tiled, int N, int K) -> Tensor", &unrepack);
}
