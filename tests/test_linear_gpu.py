"""tp.Linear / tp.matmul on the GPU at the points the reference pins with known answers, and the general
(any shape, any alignment, float32) product against the oracle.

Known answers: tripy/tests/integration/test_linear.py:27-150 (float32 Linear with in_features = 4: float, int8 and
float8 with every weight_quant_dim and with or without an input scale, int4 weight-only in four scale modes) and
mlir-tensorrt/compiler/test/python/IntegrationTests/test_tensorrt10_data_type_support.py:218-246, 304-310
(int4 dequantize -> matrix_multiply).  Each case runs through qlinear.Linear / qlinear.matmul and must equal both
the reference's expected values and the oracle's op-by-op restatement exactly."""
import numpy as np
import pytest
import torch

import oracle as orc
import qlinear as ql
from helpers import QL_OF_CODE, assert_close_rel, float_values, randn, to_np
from linear_cases import iota, linear_cases

pytestmark = pytest.mark.gpu


def _dev(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a)).to(dtype).cuda()


def test_reference_linear_known_answers(kat):
    ran = 0
    for cid, kw, want in linear_cases(kat):
        qd = QL_OF_CODE[kw["quant_code"]] if kw.get("quant_code") is not None else None
        out_f, in_f = kw["weight"].shape
        lin = ql.Linear(in_f, out_f, quant_dtype=qd, weight_quant_dim=kw.get("weight_quant_dim"))   # dtype defaults to float32
        lin.weight, lin.bias = _dev(kw["weight"]), _dev(kw["bias"])
        if qd is not None:
            lin.weight_scale = _dev(kw["weight_scale"])
            if kw.get("input_scale") is not None:
                lin.input_scale = torch.tensor(kw["input_scale"], dtype=torch.float32)
        x = _dev(kw["x"])
        if want is None:
            with pytest.raises(ql.QuantizeError, match=kat["linear_module"]["quant"]["rejected"]["message"]):
                lin(x)
        else:
            got = lin(x)
            assert got.dtype == torch.float32 and tuple(got.shape) == want.shape
            assert np.array_equal(got.cpu().numpy(), want), cid
            assert np.array_equal(got.cpu().numpy(), orc.linear_module(**kw)), cid
        ran += 1
    assert ran == 17
    torch.cuda.synchronize()


def test_default_quantized_linear_constructs_and_runs():
    lin = ql.Linear(4, 2, quant_dtype=ql.int8)
    lin.weight_scale = 1.0
    assert tuple(lin(torch.ones(3, 4, device="cuda")).shape) == (3, 2)


def test_int4_dequantize_then_matmul(kat):
    for case in kat["int4_dq_matmul"]["cases"]:
        q = ql.Int4Tensor.pack(torch.tensor(case["lhs_i4"], dtype=torch.int8).reshape(2, 2)).packed.cuda()
        lhs = ql.dequantize(ql.Int4Tensor(q, (2, 2)), case["scale"], ql.float32)
        out = ql.matmul(lhs, _dev(case["rhs"]).reshape(2, 2))
        assert out.reshape(-1).tolist() == case["expect"]


def test_matmul_rank_rules(kat):
    for case in kat["matmul_doc_examples"]["cases"]:
        a, b = iota(case["a_shape"], case["a_iota_dim"]), iota(case["b_shape"], case["b_iota_dim"])
        got = ql.matmul(_dev(a), _dev(b))
        assert tuple(got.shape) == (a @ b).shape and np.array_equal(got.cpu().numpy(), a @ b), case


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.float16, 2.0 ** -10), (torch.bfloat16, 2.0 ** -8)])
def test_matmul_broadcast_and_odd_shapes(dtype, tol):
    code = {torch.float32: orc.F32, torch.float16: orc.F16, torch.bfloat16: orc.BF16}[dtype]
    for sa, sb in [((37, 29), (29, 53)), ((3, 1, 5, 7), (2, 7, 9)), ((2, 3, 65, 130), (2, 3, 130, 67)), ((4, 6, 5), (5,)), ((5,), (4, 5, 6))]:
        a, b = randn(sa, dtype, 11), randn(sb, dtype, 12)
        got = ql.matmul(a, b)
        want = orc.to_f32(orc.matmul(to_np(a), to_np(b), code, acc64=True), code)
        assert tuple(got.shape) == want.shape
        assert_close_rel(float_values(got), want, tol, f"matmul {sa} @ {sb} {dtype}")


@pytest.mark.parametrize("M,N,K", [(3, 2, 4), (37, 53, 29), (130, 70, 100), (5, 300, 1000)])
def test_float32_linear_any_shape(M, N, K):
    x, w, b = randn((M, K), torch.float32, 21), randn((N, K), torch.float32, 22, std=0.05), randn((N,), torch.float32, 23)
    y = ql.linear(x, w, bias=b)
    want = orc.linear_float(to_np(x), to_np(w), to_np(b), orc.F32, acc64=True)
    assert_close_rel(y.cpu().numpy(), want, 1e-5, f"f32 linear {M}x{N}x{K}")


@pytest.mark.parametrize("kind", ["fp8", "int8"])
@pytest.mark.parametrize("M,N,K,out", [(3, 2, 4, torch.float32), (33, 70, 20, torch.float32), (65, 40, 72, torch.bfloat16),
                                        (48, 96, 256, torch.float32), (300, 520, 128, torch.float32)])
def test_quantized_gemm_unaligned_k_and_f32_output(kind, M, N, K, out):
    """K whose byte length is not a multiple of 16 (general kernel) and f32 results (both kernels), with per-row and
    per-channel scales and a bias, against the oracle; int8 products are exact integers, so those match bit for bit."""
    g = torch.Generator(device="cpu").manual_seed(31 + M)
    sx = (torch.rand(M, generator=g) * 0.02 + 0.01).cuda()
    sw = (torch.rand(N, generator=g) * 0.02 + 0.01).cuda()
    bias = randn((N,), torch.float32, 33)
    if kind == "fp8":
        xq = randn((M, K), torch.float32, 34).to(torch.float8_e4m3fn)
        wq = randn((N, K), torch.float32, 35).to(torch.float8_e4m3fn)
        ref = orc.gemm_fp8(to_np(xq), to_np(wq), sx.cpu().numpy(), sw.cpu().numpy(), orc.F32, acc64=True)
    else:
        xq = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8).cuda()
        wq = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8).cuda()
        ref = orc.gemm_i8(to_np(xq), to_np(wq), sx.cpu().numpy(), sw.cpu().numpy(), orc.F32)
    y = ql.linear(xq, wq, sx, sw, bias, out_dtype=QL_OF_CODE[{torch.float32: orc.F32, torch.bfloat16: orc.BF16}[out]])
    assert y.dtype == out
    want = ref.astype(np.float64) + bias.cpu().numpy().astype(np.float64)[None, :]
    tol = 1e-5 if out == torch.float32 else 2.0 ** -8
    assert_close_rel(float_values(y), want, tol, f"{kind} {M}x{N}x{K} -> {out}")
    # without bias the entry points of the quantized GEMMs take the same shapes
    y2 = (ql.gemm_fp8 if kind == "fp8" else ql.gemm_i8)(xq, wq, sx, sw, out_dtype=QL_OF_CODE[orc.F32 if out == torch.float32 else orc.BF16])
    assert_close_rel(float_values(y2), ref.astype(np.float64), tol, f"{kind} {M}x{N}x{K} no bias")
    if kind == "int8" and out == torch.float32:
        assert np.array_equal(y2.cpu().numpy(), ref)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_bias_in_the_tensor_core_epilogue(dtype):
    M, N, K = 200, 264, 320
    x, w, b = randn((M, K), dtype, 41), randn((N, K), dtype, 42, std=0.05), randn((N,), dtype, 43)
    y = ql.linear(x, w, bias=b)
    want = float_values(x).astype(np.float64) @ float_values(w).astype(np.float64).T + float_values(b).astype(np.float64)[None, :]
    assert_close_rel(float_values(y), want, 2.0 ** -10 if dtype == torch.float16 else 2.0 ** -8, f"16-bit linear with bias {dtype}")
    lin = ql.Linear(K, N, dtype=ql.float16 if dtype == torch.float16 else ql.bfloat16)
    lin.weight, lin.bias = w, b
    assert torch.equal(lin(x.reshape(2, 100, K)).reshape(M, N), y)
