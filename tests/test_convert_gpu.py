"""quantize_linears on a tiny random-weight Hugging Face Llama (no checkpoint: the container has no network):
the converted model must agree with a plain-torch model that applies the same quantisation rules step by step
(reference weight format from quantization.py / matrix_packer.py; int8 activation rule of this library)."""
import numpy as np
import pytest
import torch
from torch import nn

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _need_gpu(built_libs):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")


def _fake_quant_act(x):          # per-token int8, as sk_quantize_activation_int8 defines it
    x = x.float()
    amax = x.abs().amax(dim=-1, keepdim=True)
    s = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
    return torch.clamp(torch.round(x / s), -127, 127) * s


def _dequant_weight(weight_out_in, G):
    """float [out, in] -> the float32 values the 2-bit codes stand for (scales rounded to fp16 as the GEMM reads them)."""
    from oracle import w2a8_oracle as O
    w_kn = weight_out_in.detach().float().cpu().numpy().T.copy()
    codes, scales = O.quantize_to_uint2(w_kn, G)
    s16 = scales.astype(np.float16).astype(np.float32)
    deq = (codes.astype(np.float32) - 1.0) * np.repeat(s16, G, axis=0)
    return torch.from_numpy(deq.T.copy())


class _RefLinear(nn.Module):
    def __init__(self, linear, G):
        super().__init__()
        self.w = _dequant_weight(linear.weight, G).cuda()

    def forward(self, x):
        return (_fake_quant_act(x.to(torch.float16)) @ self.w.t()).to(torch.float16)


class _RefMLP(nn.Module):
    def __init__(self, mlp, G):
        super().__init__()
        self.gate, self.up, self.down = _RefLinear(mlp.gate_proj, G), _RefLinear(mlp.up_proj, G), _RefLinear(mlp.down_proj, G)

    def forward(self, x):
        g, u = self.gate(x).float(), self.up(x).float()
        h = g / (1.0 + torch.exp(-g)) * u
        return (_fake_quant_act(h) @ self.down.w.t()).to(torch.float16)


def _reference_model(model, G):
    import copy
    ref = copy.deepcopy(model)
    for layer in ref.model.layers:
        layer.mlp = _RefMLP(layer.mlp, G)
        for name in ("q_proj", "k_proj", "v_proj", "o_proj"):
            setattr(layer.self_attn, name, _RefLinear(getattr(layer.self_attn, name), G))
    return ref


def test_tiny_llama_swap_in_matches_step_by_step_reference():
    from transformers import LlamaConfig, LlamaForCausalLM
    from slimkernels_b200.torch import W2A8Linear, W2A8LlamaMLP, quantize_linears
    torch.manual_seed(0)
    cfg = LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=4, vocab_size=128, max_position_embeddings=64)
    model = LlamaForCausalLM(cfg).half().cuda().eval()
    G = 128
    ref = _reference_model(model, G).eval()
    stats = quantize_linears(model, group_size=G)
    assert stats == {"linear": 8, "mlp": 2, "kept": ["lm_head"]}
    assert isinstance(model.model.layers[0].mlp, W2A8LlamaMLP)
    assert isinstance(model.model.layers[1].self_attn.q_proj, W2A8Linear)
    ids = torch.randint(0, 128, (2, 24), device="cuda")
    with torch.no_grad():
        y = model(input_ids=ids).logits.float()
        y_ref = ref(input_ids=ids).logits.float()
    assert torch.isfinite(y).all()
    # same integers in both models; what differs is the order of the fp32 sums and fp16 roundings between layers
    err = (y - y_ref).abs().max().item()
    assert err <= 2e-2 * max(1.0, y_ref.abs().max().item()), err
    # decode-sized call (one token per sequence) goes through the decode kernel
    with torch.no_grad():
        y1 = model(input_ids=ids[:, :1]).logits.float()
        y1_ref = ref(input_ids=ids[:, :1]).logits.float()
    assert (y1 - y1_ref).abs().max().item() <= 2e-2 * max(1.0, y1_ref.abs().max().item())


def test_linear_with_bias_and_unconvertible_layers_are_handled():
    from slimkernels_b200.torch import quantize_linears
    torch.manual_seed(1)
    net = nn.Sequential(nn.Linear(128, 64, bias=True), nn.ReLU(), nn.Linear(64, 32)).half().cuda()
    want0 = _RefLinear(net[0], 128)
    bias = net[0].bias.detach().clone()
    stats = quantize_linears(net, group_size=128)
    assert stats["linear"] == 1 and stats["kept"] == ["2"]          # 64 input features: not a multiple of the group
    x = torch.randn(5, 128, device="cuda", dtype=torch.float16)
    with torch.no_grad():
        got = net[0](x).float()
    assert (got - (want0(x).float() + bias.float())).abs().max().item() <= 1e-2
