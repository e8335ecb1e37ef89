"""PyTorch-facing side of the W2A8 path: the op, the Linear/MLP modules and N-sharded execution."""
from .ops import (W2A8Plan, load_extension, repack_weight, unrepack_weight, w2a8_gemm,  # noqa: F401
                  w2a8_partials)
from .modules import W2A8Linear, W2A8LlamaMLP, prepare_weight_gpu, quantize_activation_int8, silu_mul_quantize_int8  # noqa: F401,E402
from .convert import quantize_linears  # noqa: F401,E402
