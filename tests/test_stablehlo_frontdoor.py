"""The StableHLO front door: programs in the three spellings the reference accepts for quantize /
dequantize (mlir-tensorrt/compiler/test/Dialect/StableHloExt/raise-qdq-*.mlir for the decomposition and
the composite, compiler/test/Passes/0_Frontend/StablehloToTensorRT/stablehlo-to-tensorrt-trt10.mlir:401-440
for the custom call) are matched on the CPU and run on the GPU against the oracle."""
import numpy as np
import pytest
import torch

import oracle as orc
import qlinear as ql
from qlinear.stablehlo import Program, UnsupportedProgram

PT_Q = """
func.func @pt_q(%arg0: tensor<48x320xf32>) -> tensor<48x320xi8> {
  %hi = stablehlo.constant dense<1.270000e+02> : tensor<f32>
  %s = stablehlo.constant dense<3.125000e-02> : tensor<f32>
  %lo = stablehlo.constant dense<-1.280000e+02> : tensor<f32>
  %0 = stablehlo.broadcast_in_dim %s, dims = [] : (tensor<f32>) -> tensor<48x320xf32>
  %1 = stablehlo.divide %arg0, %0 : tensor<48x320xf32>
  %2 = stablehlo.round_nearest_even %1 : tensor<48x320xf32>
  %3 = stablehlo.clamp %lo, %2, %hi : (tensor<f32>, tensor<48x320xf32>, tensor<f32>) -> tensor<48x320xf32>
  %4 = stablehlo.convert %3 : (tensor<48x320xf32>) -> tensor<48x320xi8>
  return %4 : tensor<48x320xi8>
}
"""

PC_Q_DQ = """
// per-channel along dim 1, then straight back
func.func @pc_round_trip(%arg0: tensor<6x3x40xf16>) -> (tensor<6x3x40xi8>, tensor<6x3x40xf16>) {
  %hi = stablehlo.constant dense<1.270000e+02> : tensor<f16>
  %lo = stablehlo.constant dense<-1.280000e+02> : tensor<f16>
  %s = stablehlo.constant dense<[2.500000e-01, 5.000000e-01, 1.250000e-01]> : tensor<3xf16>
  %0 = stablehlo.broadcast_in_dim %s, dims = [1] : (tensor<3xf16>) -> tensor<6x3x40xf16>
  %1 = stablehlo.divide %arg0, %0 : tensor<6x3x40xf16>
  %2 = stablehlo.round_nearest_even %1 : tensor<6x3x40xf16>
  %3 = stablehlo.clamp %lo, %2, %hi : (tensor<f16>, tensor<6x3x40xf16>, tensor<f16>) -> tensor<6x3x40xf16>
  %4 = stablehlo.convert %3 : (tensor<6x3x40xf16>) -> tensor<6x3x40xi8>
  %5 = stablehlo.convert %4 : (tensor<6x3x40xi8>) -> tensor<6x3x40xf16>
  %6 = stablehlo.broadcast_in_dim %s, dims = [1] : (tensor<3xf16>) -> tensor<6x3x40xf16>
  %7 = stablehlo.multiply %5, %6 : tensor<6x3x40xf16>
  return %4, %7 : tensor<6x3x40xi8>, tensor<6x3x40xf16>
}
"""

BLOCK_Q = """
func.func @block_q(%arg0: tensor<4x8xf32>) -> tensor<4x8xi4> {
  %hi = stablehlo.constant dense<7.000000e+00> : tensor<f32>
  %lo = stablehlo.constant dense<-8.000000e+00> : tensor<f32>
  %s = stablehlo.constant dense<[[5.000000e-01, 2.500000e-01, 1.000000e+00, 2.000000e+00, 5.000000e-01, 2.500000e-01, 1.000000e+00, 2.000000e+00], [1.000000e+00, 1.000000e+00, 5.000000e-01, 5.000000e-01, 2.500000e-01, 2.500000e-01, 2.000000e+00, 2.000000e+00]]> : tensor<2x8xf32>
  %0 = stablehlo.broadcast_in_dim %s, dims = [1, 2] : (tensor<2x8xf32>) -> tensor<2x2x8xf32>
  %1 = stablehlo.reshape %0 : (tensor<2x2x8xf32>) -> tensor<4x8xf32>
  %2 = stablehlo.divide %arg0, %1 : tensor<4x8xf32>
  %3 = stablehlo.round_nearest_even %2 : tensor<4x8xf32>
  %4 = stablehlo.clamp %lo, %3, %hi : (tensor<f32>, tensor<4x8xf32>, tensor<f32>) -> tensor<4x8xf32>
  %5 = stablehlo.convert %4 : (tensor<4x8xf32>) -> tensor<4x8xi4>
  return %5 : tensor<4x8xi4>
}
"""

FP8_DECOMPOSED = """
func.func @q_f8(%arg0: tensor<16x64xbf16>) -> tensor<16x64xf8E4M3FN> {
  %hi32 = stablehlo.constant dense<4.480000e+02> : tensor<f32>
  %lo32 = stablehlo.constant dense<-4.480000e+02> : tensor<f32>
  %s = stablehlo.constant dense<5.000000e-01> : tensor<bf16>
  %lo = stablehlo.convert %lo32 : (tensor<f32>) -> tensor<bf16>
  %0 = stablehlo.broadcast_in_dim %s, dims = [] : (tensor<bf16>) -> tensor<16x64xbf16>
  %1 = stablehlo.divide %arg0, %0 : tensor<16x64xbf16>
  %2 = stablehlo.round_nearest_even %1 : tensor<16x64xbf16>
  %hi = stablehlo.convert %hi32 : (tensor<f32>) -> tensor<bf16>
  %3 = stablehlo.clamp %lo, %2, %hi : (tensor<bf16>, tensor<16x64xbf16>, tensor<bf16>) -> tensor<16x64xbf16>
  %4 = stablehlo.convert %3 : (tensor<16x64xbf16>) -> tensor<16x64xf8E4M3FN>
  return %4 : tensor<16x64xf8E4M3FN>
}
"""

COMPOSITE = """
func.func @main(%arg0: tensor<32x20xf32>) -> tensor<32x20xf32> {
  %0 = stablehlo.composite "tensorrt.pc_q" %arg0 {composite_attributes = {axis = 1 : i32, scale = dense<[0.5, 0.25, 0.5, 0.25, 0.5, 0.25, 0.5, 0.25, 0.5, 0.25, 0.5, 0.25, 0.5, 0.25, 0.5, 0.25, 0.5, 0.25, 0.5, 0.25]> : tensor<20xf32>}, decomposition = @pc_q} : (tensor<32x20xf32>) -> tensor<32x20xi8>
  %1 = stablehlo.composite "tensorrt.pt_dq" %0 {composite_attributes = {axis = -1 : i32, scale = dense<2.000000e+00> : tensor<f32>}, decomposition = @pt_dq} : (tensor<32x20xi8>) -> tensor<32x20xf32>
  return %1 : tensor<32x20xf32>
}
func.func private @pc_q(%arg0: tensor<32x20xf32>) -> tensor<32x20xi8> attributes {plan.decomposition} {
  %0 = stablehlo.convert %arg0 : (tensor<32x20xf32>) -> tensor<32x20xi8>
  return %0 : tensor<32x20xi8>
}
"""

CUSTOM_CALL = """
func.func @main(%arg0: tensor<32x20xf32>, %scale: tensor<32xf32>) -> tensor<32x20xf8E4M3FN> {
  %0 = stablehlo.custom_call @tensorrt.quantize(%arg0, %scale) {api_version = 2 : i32, axis = 0 : i32, mode = "tensorrt.pc_q", operand_layouts = [dense<[1, 0]> : tensor<2xindex>, dense<0> : tensor<1xindex>], result_layouts = [dense<[1, 0]> : tensor<2xindex>]} : (tensor<32x20xf32>, tensor<32xf32>) -> tensor<32x20xf8E4M3FN>
  return %0 : tensor<32x20xf8E4M3FN>
}
"""


NVFP4 = """
func.func public @nvfp4_round_trip(%arg0: tensor<2x32xf32>, %scale: tensor<f32>) -> tensor<2x32xf32> {
  %0:2 = stablehlo.custom_call @tensorrt.dynamic_quantize(%arg0, %scale) {api_version = 2 : i32, axis = 1 : i32, block_size = 16 : i32, operand_layouts = [dense<[1, 0]> : tensor<2xindex>, dense<> : tensor<0xindex>], result_layouts = [dense<[1, 0]> : tensor<2xindex>, dense<[1, 0]> : tensor<2xindex>]} : (tensor<2x32xf32>, tensor<f32>) -> (tensor<2x32xf4E2M1FN>, tensor<2x2xf8E4M3FN>)
  %1 = stablehlo.custom_call @tensorrt.dequantize(%0#1, %scale) {api_version = 2 : i32, mode = "tensorrt.pt_dq"} : (tensor<2x2xf8E4M3FN>, tensor<f32>) -> tensor<2x2xf32>
  %2 = stablehlo.custom_call @tensorrt.dequantize(%0#0, %1) {api_version = 2 : i32, mode = "tensorrt.block_dq"} : (tensor<2x32xf4E2M1FN>, tensor<2x2xf32>) -> tensor<2x32xf32>
  return %2 : tensor<2x32xf32>
}
"""


def _linear_program(M, N, K, act="bf16"):
    """Tripy's quantized Linear as StableHLO: x @ transpose(dequantize(Wq)) with per-channel int8 weights."""
    return f"""
func.func @linear(%x: tensor<{M}x{K}x{act}>, %wq: tensor<{N}x{K}xi8>, %s: tensor<{N}x{act}>) -> tensor<{M}x{N}x{act}> {{
  %0 = stablehlo.convert %wq : (tensor<{N}x{K}xi8>) -> tensor<{N}x{K}x{act}>
  %1 = stablehlo.broadcast_in_dim %s, dims = [0] : (tensor<{N}x{act}>) -> tensor<{N}x{K}x{act}>
  %2 = stablehlo.multiply %0, %1 : tensor<{N}x{K}x{act}>
  %3 = stablehlo.transpose %2, dims = [1, 0] : (tensor<{N}x{K}x{act}>) -> tensor<{K}x{N}x{act}>
  %4 = stablehlo.dot_general %x, %3, contracting_dims = [1] x [0] : (tensor<{M}x{K}x{act}>, tensor<{K}x{N}x{act}>) -> tensor<{M}x{N}x{act}>
  return %4 : tensor<{M}x{N}x{act}>
}}
"""


# ------------------------------------------------------------------------------------------ matching (CPU)
def test_matches_per_tensor_decomposition():
    p = Program.from_text(PT_Q)
    assert p.name == "pt_q" and [s.op for s in p.steps] == ["quantize"]
    st = p.steps[0]
    assert st.attrs["mode"] == "pt" and st.attrs["axis"] is None and st.attrs["dtype"] is ql.int8
    (data, ty), = p.constants.values()
    assert ty.shape == () and float(data) == 0.03125


def test_matches_per_channel_round_trip():
    p = Program.from_text(PC_Q_DQ)
    assert [s.op for s in p.steps] == ["quantize", "dequantize"]
    assert all(s.attrs["mode"] == "pc" and s.attrs["axis"] == 1 for s in p.steps)
    assert len(p.result_slots) == 2


def test_matches_block_decomposition():
    p = Program.from_text(BLOCK_Q)
    st, = p.steps
    assert st.attrs["mode"] == "block" and st.attrs["dtype"] is ql.int4
    (data, ty), = p.constants.values()
    assert ty.shape == (2, 8)


def test_decomposed_fp8_rounds_to_integers_first():
    st, = Program.from_text(FP8_DECOMPOSED).steps
    assert st.attrs["dtype"] is ql.float8 and st.attrs["fp8_mode"] == "stablehlo"


def test_matches_composites_and_picks_the_named_function():
    p = Program.from_text(COMPOSITE, func="main")
    assert [s.op for s in p.steps] == ["quantize", "dequantize"]
    assert p.steps[0].attrs["axis"] == 1 and p.steps[0].attrs["fp8_mode"] == "direct"
    assert p.steps[1].attrs["mode"] == "pt" and p.steps[1].attrs["axis"] is None


def test_matches_custom_call_with_runtime_scale():
    p = Program.from_text(CUSTOM_CALL)
    st, = p.steps
    assert st.attrs["mode"] == "pc" and st.attrs["axis"] == 0 and st.ins == (0, 1) and not p.constants


def test_matches_nvfp4_dynamic_quantize_with_two_results():
    """Spelling of compiler/test/Passes/0_Frontend/StablehloToTensorRT/stablehlo-to-tensorrt-trt10.mlir:477-480."""
    p = Program.from_text(NVFP4)
    assert [s.op for s in p.steps] == ["dynamic_quantize", "dequantize", "dequantize"]
    dq = p.steps[0]
    assert dq.attrs["axis"] == 1 and dq.attrs["block_size"] == 16 and dq.ins == (0, 1)
    assert p.steps[1].ins[0] == dq.attrs["scales_slot"] and p.steps[2].ins == (dq.out, p.steps[1].out)
    assert p.steps[2].attrs["mode"] == "block"


def test_linear_fuses_the_dequantize_into_the_weight_only_kernel():
    p = Program.from_text(_linear_program(16, 256, 512))
    assert [s.op for s in p.steps] == ["linear_w8a16"]
    assert p.steps[0].ins == (0, 1, 2)


@pytest.mark.parametrize("text,why", [
    (PT_Q.replace("1.270000e+02", "1.000000e+02"), "clamp bounds"),
    (PT_Q.replace("stablehlo.round_nearest_even", "stablehlo.floor"), "outside the quantized-linear path"),
    (PT_Q.replace("48x320", "?x320"), "dynamic shapes"),
    (PT_Q.replace("dense<3.125000e-02>", "dense_resource<__elided__>"), "elided"),
    ("func.func @f(%a: tensor<4xf32>) -> tensor<4xf32> {\n  %0 = stablehlo.add %a, %a : tensor<4xf32>\n  return %0 : tensor<4xf32>\n}", "outside the quantized-linear path"),
])
def test_refuses_what_is_not_the_path(text, why):
    with pytest.raises(UnsupportedProgram, match=why):
        Program.from_text(text)


def test_unknown_function_name():
    with pytest.raises(UnsupportedProgram, match="not found"):
        Program.from_text(PT_Q, func="nope")


# ------------------------------------------------------------------------------------------ running (GPU)
def _np(t):
    from helpers import to_np
    return to_np(t)


@pytest.mark.gpu
def test_runs_per_tensor_quantize():
    from helpers import randn
    x = randn((48, 320), torch.float32, 501, std=2.0)
    q = Program.from_text(PT_Q)(x)
    want = orc.quantize(_np(x), orc.F32, np.float32(0.03125), orc.F32, orc.I8, orc.PER_TENSOR, None)
    assert q.dtype == torch.int8 and np.array_equal(_np(q), want)


@pytest.mark.gpu
def test_runs_per_channel_round_trip():
    from helpers import randn
    x = randn((6, 3, 40), torch.float16, 502, std=8.0)
    s = np.array([0.25, 0.5, 0.125], dtype=np.float16)
    q, y = Program.from_text(PC_Q_DQ)(x)
    want_q = orc.quantize(_np(x), orc.F16, s, orc.F16, orc.I8, orc.PER_CHANNEL, 1)
    want_y = orc.dequantize(want_q, orc.I8, s, orc.F16, orc.F16, (6, 3, 40), orc.PER_CHANNEL, 1)
    assert np.array_equal(_np(q), want_q)
    assert np.array_equal(_np(y).view(np.uint16), want_y.view(np.uint16))


@pytest.mark.gpu
def test_runs_block_quantize_to_int4():
    from helpers import randn
    x = randn((4, 8), torch.float32, 503, std=3.0)
    p = Program.from_text(BLOCK_Q)
    (data, _), = p.constants.values()
    q = p(x)
    want = orc.quantize(_np(x), orc.F32, data.astype(np.float32), orc.F32, orc.I4, orc.BLOCK, None)
    assert isinstance(q, ql.Int4Tensor) and np.array_equal(_np(q), want)


@pytest.mark.gpu
def test_runs_decomposed_fp8_with_integer_rounding():
    from helpers import randn
    x = randn((16, 64), torch.bfloat16, 504, std=20.0)
    q = Program.from_text(FP8_DECOMPOSED)(x)
    s = _np(torch.tensor(0.5, dtype=torch.bfloat16))
    want = orc.quantize(_np(x), orc.BF16, s, orc.BF16, orc.F8E4M3, orc.PER_TENSOR, None, ql._lib.FP8_MODES["stablehlo"])
    assert np.array_equal(_np(q), want)
    # the decomposition really is different from TensorRT's direct conversion on this input
    direct = orc.quantize(_np(x), orc.BF16, s, orc.BF16, orc.F8E4M3, orc.PER_TENSOR, None, ql._lib.FP8_MODES["direct"])
    assert not np.array_equal(want, direct)


@pytest.mark.gpu
def test_runs_composites():
    from helpers import randn
    x = randn((32, 20), torch.float32, 505, std=10.0)
    y = Program.from_text(COMPOSITE, func="main")(x)
    s = np.tile(np.array([0.5, 0.25], dtype=np.float32), 10)
    q = orc.quantize(_np(x), orc.F32, s, orc.F32, orc.I8, orc.PER_CHANNEL, 1)
    want = orc.dequantize(q, orc.I8, np.float32(2.0), orc.F32, orc.F32, (32, 20), orc.PER_TENSOR, None)
    assert np.array_equal(_np(y), want)


@pytest.mark.gpu
def test_runs_custom_call_with_runtime_scale():
    from helpers import randn
    x = randn((32, 20), torch.float32, 506, std=50.0)
    s = (x.abs().amax(dim=1) / 448.0).contiguous()
    q = Program.from_text(CUSTOM_CALL)(x, s)
    want = orc.quantize(_np(x), orc.F32, _np(s), orc.F32, orc.F8E4M3, orc.PER_CHANNEL, 0)
    assert np.array_equal(_np(q), want)


@pytest.mark.gpu
@pytest.mark.parametrize("M", [1, 16, 96])
def test_runs_quantized_linear(M):
    from helpers import assert_close_rel, float_values, randn
    N, K = 256, 512
    w = randn((N, K), torch.float16, 507, std=0.02)
    s = ql.amax_scale(w, ql.int8, dim=0).to(torch.bfloat16)
    wq = ql.quantize(w.to(torch.bfloat16), s, ql.int8, 0)
    x = randn((M, K), torch.bfloat16, 508)
    y = Program.from_text(_linear_program(M, N, K))(x, wq, s)
    want = orc.linear_w8(_np(x), orc.BF16, _np(wq), _np(s), orc.BF16, orc.BF16)
    assert tuple(y.shape) == (M, N)
    assert_close_rel(float_values(y), orc.to_f32(want, orc.BF16), 1e-2, "linear through the front door")


@pytest.mark.gpu
def test_runs_the_nvfp4_program_of_the_reference(kat):
    """The reference's NVFP4 execution test as a StableHLO program: same input, same expected output
    (compiler/test/python/IntegrationTests/test_tensorrt_fp4.py:10-26, 74-82)."""
    case = kat["nvfp4_dynamic_quantize"]
    x = torch.tensor(case["input"], dtype=torch.float32, device="cuda")
    gs = torch.tensor(case["double_quant_scale"], dtype=torch.float32, device="cuda")
    y = Program.from_text(NVFP4)(x, gs)
    assert np.array_equal(y.cpu().numpy(), np.array(case["expected"], dtype=np.float32))
