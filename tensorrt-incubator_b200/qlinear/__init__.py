"""qlinear: the host-side mirror of the reference's quantized-linear operators over the
B200 (sm_100a) kernels in ../csrc, reached through the C ABI in include/qlinear_b200.h."""
from ._lib import QlError, lib  # noqa: F401
from .dtypes import bfloat16, bool, float4, float8, float16, float32, int4, int8, int32, int64  # noqa: F401,A004
from .linear import Linear, gemm_16, gemm_fp8, gemm_i8, linear, linear_w4a16, linear_w8a16, matmul  # noqa: F401
from .ops import (QuantizeError, amax_scale, cast, dequantize, dequantize_nvfp4, dynamic_quantize, gemm_nvfp4, quantize,  # noqa: F401
                  quantize_dequantize, quantize_to)
from .tensor import Float4Tensor, Int4Tensor  # noqa: F401
from .mlp import (QuantizedMLP, gemm_fp8_swiglu, interleave_gate_up, quantize_per_channel_fp8, quantize_rows_fp8, rmsnorm_quant_fp8,  # noqa: F401
                  shard_range, swiglu_quant_fp8)  # noqa: F401
from . import nccl, peer, stablehlo  # noqa: F401,E402
