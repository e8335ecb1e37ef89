"""Swap the `nn.Linear` layers of a model for W2A8 layers.

The reference's torch directory wraps a Hugging Face causal LM for `generate` (slimkernels/torch/llama.py:4-47) and
stops there; this is the step it was heading towards: every linear projection of the loaded model is quantised with
the reference's own rule (quantize_to_uint2 + pack_matrix, run on the GPU) and replaced by a module that calls the
W2A8 GEMM.  Llama-style MLP blocks (gate_proj / up_proj / down_proj with SiLU) become one fused `W2A8LlamaMLP`
(gate and up share a GEMM; SiLU * up and the int8 re-quantisation are one kernel).
"""
from __future__ import annotations

import torch
from torch import nn

from .modules import W2A8Linear, W2A8LlamaMLP


class _W2A8LinearWithBias(nn.Module):
    def __init__(self, linear: W2A8Linear, bias: torch.Tensor):
        super().__init__()
        self.linear = linear
        self.register_buffer("bias", bias.detach().to(torch.float16))

    def forward(self, x):
        return self.linear(x) + self.bias


def _convertible(linear: nn.Linear, group_size: int) -> bool:
    return linear.in_features % group_size == 0 and linear.in_features % 32 == 0


def _is_llama_mlp(module: nn.Module) -> bool:
    names = ("gate_proj", "up_proj", "down_proj")
    if not all(isinstance(getattr(module, n, None), nn.Linear) for n in names):
        return False
    if any(getattr(module, n).bias is not None for n in names):
        return False
    act = getattr(module, "act_fn", None)
    return isinstance(act, nn.SiLU) or type(act).__name__ in ("SiLU", "SiLUActivation")


def quantize_linears(model: nn.Module, group_size: int = 128, skip=("lm_head",), fuse_mlp: bool = True,
                     device=None) -> dict:
    """Replace, in place, every `nn.Linear` whose in_features is a multiple of `group_size` (except names in `skip`).

    Returns {"linear": n, "mlp": n, "kept": [names left as they were]}.  The model must be on a CUDA device (or
    `device` given): quantisation runs there.
    """
    stats = {"linear": 0, "mlp": 0, "kept": []}

    def dev_of(linear):
        return device if device is not None else linear.weight.device

    def convert(linear: nn.Linear):
        q = W2A8Linear.from_float(linear.weight, group_size, device=dev_of(linear))
        return q if linear.bias is None else _W2A8LinearWithBias(q, linear.bias.to(dev_of(linear)))

    def walk(parent: nn.Module, prefix: str):
        for name, child in list(parent.named_children()):
            full = f"{prefix}{name}"
            if name in skip or full in skip:
                stats["kept"].append(full)
                continue
            if fuse_mlp and _is_llama_mlp(child) and _convertible(child.gate_proj, group_size) \
                    and _convertible(child.down_proj, group_size):
                gate_up = torch.cat([child.gate_proj.weight, child.up_proj.weight], dim=0)   # gate rows first
                fused = W2A8LlamaMLP(W2A8Linear.from_float(gate_up, group_size, device=dev_of(child.gate_proj)),
                                     W2A8Linear.from_float(child.down_proj.weight, group_size,
                                                           device=dev_of(child.down_proj)))
                setattr(parent, name, fused)
                stats["mlp"] += 1
            elif isinstance(child, nn.Linear):
                if _convertible(child, group_size):
                    setattr(parent, name, convert(child))
                    stats["linear"] += 1
                else:
                    stats["kept"].append(full)
            else:
                walk(child, full + ".")

    walk(model, "")
    return stats
