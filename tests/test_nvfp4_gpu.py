"""NVFP4 (tensorrt.dynamic_quantize and its inverse) on the GPU against the oracle: e2m1 data and e4m3 block
scales bit for bit, the dequantized values bit for bit; the reference's own known answer
(compiler/test/python/IntegrationTests/test_tensorrt_fp4.py:74-82) through the C ABI."""
import numpy as np
import pytest
import torch

import oracle as orc
import qlinear as ql
from helpers import code_of, randn, to_np

pytestmark = pytest.mark.gpu


def test_reference_known_answer(kat):
    case = kat["nvfp4_dynamic_quantize"]
    x = torch.tensor(case["input"], dtype=torch.float32, device="cuda")
    data, scales = ql.dynamic_quantize(x, case["double_quant_scale"], axis=1)
    assert data.shape == (2, 32) and tuple(scales.shape) == (2, 2)
    y = ql.dequantize_nvfp4(data, scales, case["double_quant_scale"], ql.float32)
    assert np.array_equal(y.cpu().numpy(), np.array(case["expected"], dtype=np.float32))
    assert torch.equal(data.unpack() * scales.float().repeat_interleave(16, dim=1), y)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape,gscale", [((7, 48), 1.0), ((3, 5, 160), 0.25), ((1024, 4096), 2.0), ((16,), 1.0)])
def test_matches_oracle(dtype, shape, gscale):
    x = randn(shape, dtype, 900 + len(shape), std=3.0)
    data, scales = ql.dynamic_quantize(x, gscale)
    want_q, want_s = orc.dynamic_quantize_nvfp4(to_np(x), code_of(x), gscale)
    assert np.array_equal(to_np(scales), want_s)
    assert np.array_equal(data.packed.cpu().numpy().reshape(want_q.shape), want_q)
    for out in (ql.float32, dtype and ql.dtypes.from_torch(dtype)):
        y = ql.dequantize_nvfp4(data, scales, gscale, out)
        want_y = orc.dequantize_nvfp4(want_q, want_s, gscale, out.code)
        assert np.array_equal(to_np(y).view(np.uint8), want_y.view(np.uint8))


def test_edge_values():
    # zeros (scale rounds to zero -> zeros), ties, saturation, a huge block and a tiny one next to each other
    x = torch.zeros((4, 32), device="cuda")
    x[1, :16] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0])
    x[2, :16] = 1e30
    x[2, 16:] = 1e-30
    x[3, 5] = float("inf")
    data, scales = ql.dynamic_quantize(x, 1.0)
    want_q, want_s = orc.dynamic_quantize_nvfp4(x.cpu().numpy(), orc.F32, 1.0)
    assert np.array_equal(to_np(scales), want_s)
    assert np.array_equal(data.packed.cpu().numpy().reshape(want_q.shape), want_q)
    assert torch.equal(data.unpack()[0], torch.zeros(32, device="cuda"))
    # block of row 1: scale 1 exactly, so the e2m1 rounding is visible: ties to even
    assert data.unpack()[1, :8].tolist() == [0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0]


def test_argument_rules():
    x = torch.ones((4, 24), device="cuda")
    with pytest.raises(ql.QlError, match="must be divisible by 16"):
        ql.dynamic_quantize(x)
    with pytest.raises(ql.QlError, match="only block size of 16"):
        ql.dynamic_quantize(torch.ones((4, 32), device="cuda"), block_size=32)
    with pytest.raises(ql.QlError, match="invalid axis"):
        ql.dynamic_quantize(torch.ones((2, 4, 32), device="cuda"), axis=0)
    with pytest.raises(ql.QlError, match="second last dimension are not built"):
        ql.dynamic_quantize(torch.ones((32, 32), device="cuda"), axis=0)


def test_reference_program_as_written(kat):
    """The reference's test program step by step: dynamic_quantize, tensorrt.dequantize of the e4m3 block scales by
    the per-tensor scale, tensorrt.dequantize of the e2m1 data by those scales
    (compiler/test/python/IntegrationTests/test_tensorrt_fp4.py:20-24)."""
    case = kat["nvfp4_dynamic_quantize"]
    x = torch.tensor(case["input"], dtype=torch.float32, device="cuda")
    data, scales = ql.dynamic_quantize(x, 1.0, axis=1)
    block_scales = ql.dequantize(scales, 1.0, ql.float32)
    assert tuple(block_scales.shape) == (2, 2)
    y = ql.dequantize(data, block_scales, ql.float32)
    assert np.array_equal(y.cpu().numpy(), np.array(case["expected"], dtype=np.float32))


@pytest.mark.parametrize("out", [ql.float32, ql.float16, ql.bfloat16])
@pytest.mark.parametrize("block", [16, 32, 64])
def test_f4_dequantize_with_float_block_scales(out, block):
    x = randn((33, 192), torch.float32, 950, std=2.0)
    data, _ = ql.dynamic_quantize(x, 1.0)
    s = (torch.rand((33, 192 // block), generator=torch.Generator().manual_seed(3)) + 0.25).to(out.torch).cuda()
    y = ql.dequantize(data, s, out)
    want = (data.unpack() * s.float().repeat_interleave(block, dim=1)).to(out.torch)   # one f32 multiply, one rounding
    assert torch.equal(y, want)
    with pytest.raises(ql.QlError, match="multiple of 16"):
        ql.dequantize(data, torch.ones((33, 24), device="cuda"), ql.float32)


@pytest.mark.parametrize("M,N,K", [(128, 128, 256), (64, 96, 64), (200, 136, 320), (512, 384, 1024), (1000, 1100, 2080)])
@pytest.mark.parametrize("out", [torch.float32, torch.bfloat16])
def test_block_scaled_gemm_matches_dequantize_then_matmul(M, N, K, out):
    """tcgen05.mma kind::mxf4nvf4 with the block scales in tensor memory against the oracle's dequantize -> f64
    product of the very same quantized operands (row, column and k tails; K not a multiple of the 256-element k step).
    The tensor core multiplies exact e2m1 products by the block scales and accumulates in f32, so the result is held
    to the f32 accumulation bound (and to the result type's rounding step)."""
    a, b = randn((M, K), torch.float32, 950 + M, std=2.0), randn((N, K), torch.float32, 951 + N, std=0.5)
    ga, gb = 0.5, 2.0
    qa, sa = ql.dynamic_quantize(a, ga)
    qb, sb = ql.dynamic_quantize(b, gb)
    y = ql.gemm_nvfp4(qa, sa, qb, sb, ga, gb, out_dtype=ql.dtypes.from_torch(out))
    assert ql.lib().ql_gemm_status(None) == 0
    want = orc.gemm_nvfp4(qa.packed.cpu().numpy().reshape(M, K // 2), to_np(sa), ga, qb.packed.cpu().numpy().reshape(N, K // 2), to_np(sb), gb)
    got = y.double().cpu().numpy()
    scale = np.sqrt(np.mean(want * want))
    tol = 2e-5 if out == torch.float32 else 2.0 ** -8
    assert np.all(np.abs(got - want) <= tol * np.maximum(np.abs(want), scale)), float(np.abs(got - want).max() / scale)
    # and it agrees with the library's own dequantize -> general product route within the benchmark's bound
    ref = ql.linear(ql.dequantize_nvfp4(qa, sa, ga, ql.float32), ql.dequantize_nvfp4(qb, sb, gb, ql.float32))
    assert float((y.float() - ref).abs().max() / ref.abs().max()) < 1e-2


@pytest.mark.parametrize("M,N,K", [(256, 224, 256), (200, 136, 320), (512, 384, 1024), (1000, 1100, 2080), (129, 100, 64), (2048, 4096, 512)])
@pytest.mark.parametrize("out", [torch.float32, torch.bfloat16])
def test_block_scaled_gemm_on_cta_pairs(M, N, K, out, monkeypatch):
    """The CTA-pair kernel (256 x 224 tiles, tcgen05.mma.cta_group::2, each CTA with its own rows of A and half of B and
    the scales of both in its tensor memory), forced for shapes that would otherwise take the one-CTA kernel: against
    the oracle as above (row tails inside the second CTA's half, column tails in either half of the B tile, k tails),
    and bit for bit against the one-CTA kernel, which adds the same products in the same order."""
    a, b = randn((M, K), torch.float32, 960 + M, std=2.0), randn((N, K), torch.float32, 961 + N, std=0.5)
    ga, gb = 0.5, 2.0
    qa, sa = ql.dynamic_quantize(a, ga)
    qb, sb = ql.dynamic_quantize(b, gb)
    results = {}
    for choice in ("pair", "one"):
        monkeypatch.setenv("QL_NVFP4_KERNEL", choice)
        ql.lib().ql_reload_tuning()
        try:
            y = torch.full((M, N), float("nan"), dtype=out, device="cuda")
            ql.gemm_nvfp4(qa, sa, qb, sb, ga, gb, out_dtype=ql.dtypes.from_torch(out), out=y)
            torch.cuda.synchronize()
            results[choice] = y
        finally:
            monkeypatch.delenv("QL_NVFP4_KERNEL")
            ql.lib().ql_reload_tuning()
    assert ql.lib().ql_gemm_status(None) == 0
    want = orc.gemm_nvfp4(qa.packed.cpu().numpy().reshape(M, K // 2), to_np(sa), ga, qb.packed.cpu().numpy().reshape(N, K // 2), to_np(sb), gb)
    got = results["pair"].double().cpu().numpy()
    scale = np.sqrt(np.mean(want * want))
    tol = 2e-5 if out == torch.float32 else 2.0 ** -8
    assert np.all(np.abs(got - want) <= tol * np.maximum(np.abs(want), scale)), float(np.abs(got - want).max() / scale)
    assert torch.equal(results["pair"], results["one"])


def test_block_scaled_gemm_argument_rules():
    qa, sa = ql.dynamic_quantize(torch.ones((4, 48), device="cuda"))
    qb, sb = ql.dynamic_quantize(torch.ones((8, 48), device="cuda"))
    with pytest.raises(ql.QlError, match="multiple of 32"):
        ql.gemm_nvfp4(qa, sa, qb, sb)
    qc, sc = ql.dynamic_quantize(torch.ones((8, 64), device="cuda"))
    qd, sd = ql.dynamic_quantize(torch.ones((4, 64), device="cuda"))
    with pytest.raises(ql.QlError, match="one entry per block of 16"):
        ql.gemm_nvfp4(qd, sc, qc, sc)
    with pytest.raises(ql.QlError, match="inner dimensions differ"):
        ql.gemm_nvfp4(qa, sa, qc, sc)
    assert tuple(ql.gemm_nvfp4(qd, sd, qc, sc, out_dtype=ql.float32).shape) == (4, 8)
