"""nn.Module wrappers: W2A8Linear and the Llama MLP block (benchmark config 4).

The reference's torch directory only wraps Hugging Face `generate` (slimkernels/torch/llama.py:4-47) and holds
no quantised layer; these modules are what would replace `nn.Linear` / `LlamaMLP` there.
"""
from __future__ import annotations

import torch
from torch import nn

from .ops import W2A8Plan, load_extension


def quantize_activation_int8(x):
    """Per-token symmetric int8: s = max|x|/127 (1.0 for an all-zero row), q = clamp(rint(x/s), -127, 127).
    x float16 [M, K] (CUDA) -> (int8 [M, K], float32 [M])."""
    load_extension()
    return torch.ops.slimkernels.quantize_activation_int8(x)


def silu_mul_quantize_int8(gate_up):
    """gate_up float16 [M, 2I] (gate first) -> int8 quantisation of SiLU(gate) * up: (int8 [M, I], float32 [M])."""
    load_extension()
    return torch.ops.slimkernels.silu_mul_quantize_int8(gate_up)


def prepare_weight_gpu(weight_kn, group_size=128):
    """float32 W[K, N] (CUDA) -> (w_packed uint8 [N, K/4], w_scale float16 [K/G, N]) on the GPU: the same bits as
    format.prepare_weight, i.e. the reference's quantize_to_uint2 (quantization.py:3) + pack_matrix
    (matrix_packer.py:3) on the transposed codes."""
    load_extension()
    packed, s16, _ = torch.ops.slimkernels.w2a8_quantize_weight(weight_kn.contiguous(), group_size)
    return packed, s16


class W2A8Linear(nn.Module):
    """y = dequant(w_packed, w_scale) applied to dynamically int8-quantised activations.

    w_packed uint8 [out_features, in_features/4] (matrix_packer layout), w_scale float16 [in_features/G, out_features].
    """

    def __init__(self, w_packed, w_scale, group_size=128, zero_point=1, out_dtype=torch.float16):
        super().__init__()
        self.register_buffer("w_packed", w_packed, persistent=True)
        self.register_buffer("w_scale", w_scale, persistent=True)
        self.group_size, self.zero_point, self.out_dtype = group_size, zero_point, out_dtype
        self.out_features, self.in_features = w_packed.shape[0], w_packed.shape[1] * 4
        self._plan, self._plan_key = None, None

    @classmethod
    def from_float(cls, weight_out_in, group_size=128, device="cuda", out_dtype=torch.float16):
        """Quantise a float weight [out_features, in_features] with the reference's rule, on the GPU."""
        w_kn = weight_out_in.detach().to(device=device, dtype=torch.float32).t().contiguous()
        w_packed, w_scale = prepare_weight_gpu(w_kn, group_size)
        return cls(w_packed, w_scale, group_size, 1, out_dtype)

    def plan(self) -> W2A8Plan:
        """The plan of the CURRENT weight buffers: it holds a tiled copy of w_packed and a pointer to w_scale, so it
        is rebuilt when the buffers were written in place (load_state_dict) or replaced (.to(), .cuda())."""
        key = (self.w_packed.data_ptr(), self.w_packed._version, self.w_scale.data_ptr(), self.w_scale._version,
               self.w_packed.device)
        if self._plan is None or self._plan_key != key:
            self._plan = W2A8Plan(self.w_packed, self.w_scale, group_size=self.group_size, zero_point=self.zero_point,
                                  out_dtype=self.out_dtype)
            self._plan_key = key
        return self._plan

    def forward_quantized(self, x_q, x_scale):
        return self.plan().gemm(x_q, x_scale)

    def forward(self, x):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).to(torch.float16)
        x_q, x_scale = quantize_activation_int8(x2)
        return self.plan().gemm(x_q, x_scale).reshape(*shape[:-1], self.out_features)


class W2A8LlamaMLP(nn.Module):
    """down( SiLU(gate(x)) * up(x) ) with W2A8 projections; gate and up are one fused [2*inter, hidden] weight
    (gate rows first).  Four kernels per call: quantise, GEMM, SiLU*up + re-quantise, GEMM."""

    def __init__(self, gate_up: W2A8Linear, down: W2A8Linear):
        super().__init__()
        assert gate_up.out_features == 2 * down.in_features and down.out_features == gate_up.in_features
        assert gate_up.out_dtype == torch.float16
        self.gate_up, self.down = gate_up, down

    def forward(self, x):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).to(torch.float16)
        gate_up_plan, down_plan = self.gate_up.plan(), self.down.plan()      # also loads the extension
        y = torch.ops.slimkernels.w2a8_mlp_forward(gate_up_plan._h, down_plan._h, x2,
                                                   self.down.out_features, self.down.out_dtype == torch.bfloat16)
        return y.reshape(*shape[:-1], self.down.out_features)
