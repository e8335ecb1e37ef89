"""Helpers for the GPU parity tests: device buffers through torch, compute through the C ABI (ctypes)."""
import numpy as np
import torch

from slimkernels_b200 import capi


class DeviceProblem:
    """Uploads one GEMM's operands and owns a C-ABI plan for the weight."""

    def __init__(self, x_q, x_scale, w_packed, w_scale, group_size=128, zero_point=1, out_dtype=torch.float16,
                 device="cuda:0", ld_x=None):
        self.dev = torch.device(device)
        self.M, self.K = x_q.shape
        self.N = w_packed.shape[0]
        self.G, self.zp, self.out_dtype = group_size, zero_point, out_dtype
        ld_x = ld_x or self.K
        xbuf = torch.zeros(self.M, ld_x, dtype=torch.int8, device=self.dev)
        xbuf[:, :self.K] = torch.from_numpy(x_q).to(self.dev)
        self.x_q, self.ld_x = xbuf, ld_x
        self.x_scale = torch.from_numpy(x_scale).to(self.dev)
        self.w_packed = torch.from_numpy(w_packed).to(self.dev)
        self.w_scale = torch.from_numpy(w_scale).to(self.dev)
        self.plan = capi.Plan(self.dev.index or 0, self.N, self.K, group_size, zero_point,
                              self.w_packed.data_ptr(), self.w_scale.data_ptr(),
                              capi.SK_OUT_BF16 if out_dtype == torch.bfloat16 else capi.SK_OUT_F16)

    def stream(self):
        return torch.cuda.current_stream(self.dev).cuda_stream

    def gemm(self, ld_out=None, M=None):
        M = M or self.M
        ld_out = ld_out or self.N
        out = torch.full((M, ld_out), float("nan"), dtype=self.out_dtype, device=self.dev)
        self.plan.gemm(M, self.x_q.data_ptr(), self.ld_x, self.x_scale.data_ptr(), out.data_ptr(), ld_out,
                       self.stream())
        torch.cuda.synchronize(self.dev)
        assert self.plan.device_status() == 0
        return out

    def partials(self):
        out = torch.full((self.K // self.G, self.M, self.N), -(2 ** 31), dtype=torch.int32, device=self.dev)
        self.plan.partials(self.M, self.x_q.data_ptr(), self.ld_x, out.data_ptr(), self.stream())
        torch.cuda.synchronize(self.dev)
        assert self.plan.device_status() == 0
        return out

    def force(self, kernel=0, token_tile=0, split_k=0, persistent=0, dependent_launch=0, tma_store=0):
        self.plan.set_option(capi.SK_OPT_KERNEL, kernel)
        self.plan.set_option(capi.SK_OPT_TOKEN_TILE, token_tile)
        self.plan.set_option(capi.SK_OPT_SPLIT_K, split_k)
        self.plan.set_option(capi.SK_OPT_PERSISTENT, persistent)
        self.plan.set_option(capi.SK_OPT_DEPENDENT_LAUNCH, dependent_launch)
        self.plan.set_option(capi.SK_OPT_TMA_STORE, tma_store)
        return self


def to_np(t):
    return t.detach().float().cpu().numpy() if t.is_floating_point() else t.detach().cpu().numpy()


def random_problem(M, N, K, G=128, seed=0):
    rng = np.random.default_rng(seed)
    x_q = rng.integers(-127, 128, size=(M, K), dtype=np.int8)
    x_scale = rng.uniform(0.005, 0.02, size=(M,)).astype(np.float32)
    w_packed = rng.integers(0, 256, size=(N, K // 4), dtype=np.uint8)
    w_scale = rng.uniform(0.001, 0.01, size=(K // G, N)).astype(np.float16)
    return x_q, x_scale, w_packed, w_scale
