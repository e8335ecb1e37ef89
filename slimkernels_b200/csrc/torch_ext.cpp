// PyTorch C++ extension: marshals tensors into the C ABI of include/sk_w2a8.h.  No kernels live here.
// Registers the ops of namespace `slimkernels` used by slimkernels_b200/torch/ops.py.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/types.h>

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

}  // namespace

TORCH_LIBRARY(slimkernels, m) {
  m.def("w2a8_plan_create(Tensor w, Tensor w_scale, int N, int K, int group_size, int zero_point, bool bf16_out, bool tiled) -> int", &plan_create);
  m.def("w2a8_plan_destroy(int plan) -> ()", &plan_destroy);
  m.def("w2a8_plan_set_option(int plan, int key, int value) -> ()", &plan_set_option);
  m.def("w2a8_plan_gemm(int plan, Tensor x_q, Tensor x_scale, int N, int K, bool bf16_out) -> Tensor", &gemm);
  m.def("w2a8_plan_gemm_out(int plan, Tensor x_q, Tensor x_scale, Tensor(a!) out, int K) -> ()", &gemm_out);
  m.def("w2a8_plan_gemm_scatter(int plan, Tensor x_q, Tensor x_scale, int[] out_ptrs, int ld_out, int col_offset, int K) -> ()", &gemm_scatter);
  m.def("w2a8_plan_partials(int plan, Tensor x_q, int N, int K, int group_size) -> Tensor", &partials);
  m.def("w2a8_plan_device_status(int plan) -> int", &device_status);
  m.def("quantize_activation_int8(Tensor x) -> (Tensor, Tensor)", &quantize_activation);
  m.def("w2a8_quantize_weight(Tensor w_kn, int group_size) -> (Tensor, Tensor, Tensor)", &quantize_weight);
  m.def("silu_mul_quantize_int8(Tensor gate_up) -> (Tensor, Tensor)", &silu_mul_quantize);
  m.def("w2a8_mlp_forward(int gate_up_plan, int down_plan, Tensor x, int hidden_out, bool bf16_out) -> Tensor", &mlp_forward);
  m.def("w2a8_repack(Tensor w_packed) -> Tensor", &repack);
  m.def("w2a8_unrepack(Tensor w_tiled, int N, int K) -> Tensor", &unrepack);
}
