"""The quantized MLP block (benchmark config 5) on one GPU against the oracle pipeline.
RMSNorm+quantize must match the oracle bit for bit (same f32 arithmetic, f64 mean); the SwiGLU
stage uses the GPU's expf, so its e4m3 output may differ from the host libm's in isolated
elements by one e4m3 step, and the block output is held to the benchmark's 1e-2 relative bound.

The block exists in two arrangements with their own oracle restatements: SwiGLU as a row kernel over the
projection rounded to the activation type, and SwiGLU in the gate/up projection's epilogue (from the unrounded
f32 sums; the product rounded once to the activation type, then quantized per row).  Neither is a reference
operator; both are held to the same bound against their restatement and to the fp8 noise floor against the
unquantized block."""
import numpy as np
import pytest
import torch

import oracle as orc
import qlinear as ql
from helpers import assert_close_rel, float_values, randn, to_np

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,code", [(torch.bfloat16, orc.BF16), (torch.float16, orc.F16)])
@pytest.mark.parametrize("T,H", [(7, 256), (64, 8192), (33, 1040), (5, 4096), (3, 12288), (4, 8208)])
def test_rmsnorm_quant_matches_oracle(dtype, code, T, H):
    x = randn((T, H), dtype, 600 + T)
    q, s = ql.rmsnorm_quant_fp8(x, 1e-5)
    wq, ws = orc.rmsnorm_quant_fp8(to_np(x), code, 1e-5)
    assert np.array_equal(to_np(s), ws)
    assert np.array_equal(to_np(q), wq)


@pytest.mark.parametrize("T,I", [(5, 128), (32, 3584), (16, 1008)])
def test_swiglu_quant_matches_oracle(T, I):
    gu = randn((T, 2 * I), torch.bfloat16, 610 + T, std=2.0)
    q, s = ql.swiglu_quant_fp8(gu)
    wq, ws = orc.swiglu_quant_fp8(to_np(gu), orc.BF16)
    assert np.allclose(to_np(s), ws, rtol=2e-6)
    got, want = orc.f8_to_f32(to_np(q)), orc.f8_to_f32(wq)
    # one e4m3 step is 2^-3 relative; differences may only be isolated boundary cases
    assert np.mean(got != want) < 1e-3
    assert np.all(np.abs(got - want) <= 0.126 * np.maximum(np.abs(want), 2.0 ** -6))


def _oracle_mlp(x, wg, wu, wd, code, fused=True):
    """The block on the host: every stage through the oracle, weights quantized per output channel."""
    def qpc(w):
        w = to_np(w) if isinstance(w, torch.Tensor) else w
        am = orc.amax(w, code, orc.PER_CHANNEL, 0)
        s = orc.scale_from_amax(am, 448.0, orc.F32)
        return orc.quantize(w, code, s, orc.F32, orc.F8E4M3, orc.PER_CHANNEL, 0), s
    wq_d, s_d = qpc(wd)
    xq, sx = orc.rmsnorm_quant_fp8(to_np(x), code, 1e-5)
    if fused:
        wq_gu, s_gu = qpc(orc.interleave_gate_up(to_np(wg), to_np(wu)))
        act, am = orc.gemm_fp8_swiglu(xq, wq_gu, sx, s_gu, code)
        aq, sa = orc.quantize_rows_fp8(act, code, am)
    else:
        wq_gu, s_gu = qpc(torch.cat([wg, wu], 0))
        gu = orc.gemm_fp8(xq, wq_gu, sx, s_gu, code)
        aq, sa = orc.swiglu_quant_fp8(gu, code)
    return orc.to_f32(orc.gemm_fp8(aq, wq_d, sa, s_d, code), code)


@pytest.mark.parametrize("dtype,code", [(torch.bfloat16, orc.BF16), (torch.float16, orc.F16)])
@pytest.mark.parametrize("M,I,K", [(200, 128, 256), (70, 96, 144), (512, 512, 512), (1000, 1792, 384)])
def test_gate_up_projection_with_swiglu_epilogue(dtype, code, M, I, K):
    """One-CTA kernel (small shapes) and CTA-pair kernel (M > 256, N >= 512): act against the oracle within the
    activation type's rounding step (the GPU's fast exponential moves isolated values by one step), row maxima
    exactly the maxima of the act the kernel wrote, and the row quantize bit for bit."""
    g = torch.Generator(device="cpu").manual_seed(640 + M)
    xq = torch.randn((M, K), generator=g).to(torch.float8_e4m3fn).cuda()
    w = ql.interleave_gate_up((torch.randn((I, K), generator=g) * 0.5).cuda(), (torch.randn((I, K), generator=g) * 0.5).cuda())
    wq = w.to(torch.float8_e4m3fn)
    sx = (torch.rand(M, generator=g) * 0.5 + 0.5).cuda()
    sw = (torch.rand(2 * I, generator=g) * 0.5 + 0.25).cuda()   # projections of order one: the exponential matters
    act = torch.full((M, I), float("nan"), dtype=dtype, device="cuda")
    amax = torch.full((M,), -1.0, dtype=torch.float32, device="cuda")
    ql.gemm_fp8_swiglu(xq, wq, sx, sw, act, amax)
    assert ql.lib().ql_gemm_status(None) == 0
    want, _ = orc.gemm_fp8_swiglu(to_np(xq), to_np(wq), sx.cpu().numpy(), sw.cpu().numpy(), code)
    step = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -9
    assert_close_rel(float_values(act), orc.to_f32(want, code), step, f"swiglu epilogue {M}x{I}x{K}")
    assert torch.equal(amax, act.float().abs().amax(dim=1))
    q, s = ql.quantize_rows_fp8(act, amax)
    wq_rows, ws = orc.quantize_rows_fp8(to_np(act), code, amax.cpu().numpy())
    assert np.array_equal(to_np(s), ws) and np.array_equal(to_np(q), wq_rows)


@pytest.mark.parametrize("dtype,code", [(torch.bfloat16, orc.BF16), (torch.float16, orc.F16)])
@pytest.mark.parametrize("T,I", [(5, 4096), (3, 28672), (2, 16400), (6, 4112), (9, 240)])
def test_row_quantize_matches_oracle(dtype, code, T, I):
    """Long rows take the kernel that walks one row segment per block (a ragged last segment and a row length that
    is not a multiple of the block's stride among the cases), short rows the flat one: bit for bit."""
    act = randn((T, I), dtype, 650 + T, std=1.5)
    act[1, :] = 0
    amax = act.float().abs().amax(dim=1)
    q, s = ql.quantize_rows_fp8(act, amax)
    wq, ws = orc.quantize_rows_fp8(to_np(act), code, amax.cpu().numpy())
    assert np.array_equal(to_np(s), ws) and np.array_equal(to_np(q), wq)


def test_row_quantize_handles_zero_rows():
    act = torch.zeros((3, 32), dtype=torch.bfloat16, device="cuda")
    act[1, 5] = -3.0
    amax = act.float().abs().amax(dim=1)
    q, s = ql.quantize_rows_fp8(act, amax)
    assert s.tolist() == [1.0, float(np.float32(3.0) / np.float32(448.0)), 1.0]
    assert float(q.float()[1, 5]) == -448.0 and float(q.float().abs().sum()) == 448.0


def test_swiglu_epilogue_refuses_what_the_tensor_cores_cannot_take():
    xq = torch.zeros((4, 24), dtype=torch.float8_e4m3fn, device="cuda")
    wq = torch.zeros((64, 24), dtype=torch.float8_e4m3fn, device="cuda")
    one = torch.ones((), device="cuda")
    with pytest.raises(ql.QlError, match="multiple of 16"):
        ql.gemm_fp8_swiglu(xq, wq, one, one, torch.empty((4, 32), dtype=torch.bfloat16, device="cuda"), torch.empty(4, device="cuda"))


def test_block_matches_oracle_pipeline():
    T, H, I = 48, 256, 512
    x = randn((T, H), torch.bfloat16, 620)
    wg, wu = randn((I, H), torch.bfloat16, 621, 0.05), randn((I, H), torch.bfloat16, 622, 0.05)
    wd = randn((H, I), torch.bfloat16, 623, 0.05)
    xf = x.double()
    r = xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + 1e-5)
    ref = (torch.nn.functional.silu(r @ wg.double().T) * (r @ wu.double().T)) @ wd.double().T
    for fused in (True, False):
        mlp = ql.QuantizedMLP(wg, wu, wd, fused_swiglu=fused)
        assert mlp.fused_swiglu == fused
        y = mlp(x)
        want = _oracle_mlp(x, wg, wu, wd, orc.BF16, fused)
        assert_close_rel(float_values(y), want, 1e-2, f"mlp block, swiglu in the epilogue: {fused}")
        # and close to the unquantized block (fp8 noise only)
        err = (y.double() - ref).abs().max() / ref.abs().max()
        assert float(err) < 0.08


def test_column_row_split_sums_to_the_unsharded_block():
    """Two shards computed one after the other on one GPU: gate/up split by columns, down by rows;
    their partial outputs summed in f32 agree with the unsharded block up to the per-shard
    activation scales (each shard re-quantizes its own columns)."""
    T, H, I = 32, 256, 1024
    x = randn((T, H), torch.bfloat16, 630)
    wg, wu = randn((I, H), torch.bfloat16, 631, 0.05), randn((I, H), torch.bfloat16, 632, 0.05)
    wd = randn((H, I), torch.bfloat16, 633, 0.05)
    full = ql.QuantizedMLP(wg, wu, wd)(x).float()
    parts = []
    for rank in range(2):
        a, b = ql.shard_range(I, 2, rank)
        parts.append(ql.QuantizedMLP(wg[a:b].contiguous(), wu[a:b].contiguous(), wd[:, a:b].contiguous())(x).float().clone())
    # each shard re-quantizes with its own per-token scale, so the two results differ by fp8 rounding
    # noise (one e4m3 step is up to 6 % of a value); compare in the Frobenius norm
    total = (parts[0] + parts[1]).double()
    rel = float((total - full.double()).norm() / full.double().norm())
    assert rel < 0.06, rel


def test_config5_full_size_first_tokens_against_the_oracle():
    """Config 5 at its full size (4096 tokens, 8192 -> 28672 -> 8192): the GPU runs the whole block; the oracle runs
    the same weights on the first and the last four tokens (every token's result depends on all of both weight
    matrices, so these rows exercise every column tile of both GEMMs)."""
    T, H, I = 4096, 8192, 28672
    g = torch.Generator(device="cuda").manual_seed(1005)
    def w(shape):
        return (torch.randn(shape, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    wg, wu, wd = w((I, H)), w((I, H)), w((H, I))
    x = torch.randn((T, H), generator=g, device="cuda").to(torch.bfloat16)
    mlp = ql.QuantizedMLP(wg, wu, wd)
    y = mlp(x)
    assert ql.lib().ql_gemm_status(None) == 0
    rows = torch.cat([x[:4], x[-4:]]).contiguous()
    want = _oracle_mlp(rows, wg, wu, wd, orc.BF16)
    got = torch.cat([y[:4], y[-4:]])
    assert_close_rel(float_values(got), want, 1e-2, "config 5 full size")
