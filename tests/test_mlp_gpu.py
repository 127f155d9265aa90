"""The quantized MLP block (benchmark config 5) on one GPU against the oracle pipeline.
RMSNorm+quantize must match the oracle bit for bit (same f32 arithmetic, f64 mean); the SwiGLU
stage uses the GPU's expf, so its e4m3 output may differ from the host libm's in isolated
elements by one e4m3 step, and the block output is held to the benchmark's 1e-2 relative bound."""
import numpy as np
import pytest
import torch

import oracle as orc
import qlinear as ql
from helpers import assert_close_rel, float_values, randn, to_np

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,code", [(torch.bfloat16, orc.BF16), (torch.float16, orc.F16)])
@pytest.mark.parametrize("T,H", [(7, 256), (64, 8192), (33, 1040)])
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


def _oracle_mlp(x, wg, wu, wd, code):
    """The block on the host: every stage through the oracle, weights quantized per output channel."""
    def qpc(w):
        am = orc.amax(to_np(w), code, orc.PER_CHANNEL, 0)
        s = orc.scale_from_amax(am, 448.0, orc.F32)
        return orc.quantize(to_np(w), code, s, orc.F32, orc.F8E4M3, orc.PER_CHANNEL, 0), s
    wq_gu, s_gu = qpc(torch.cat([wg, wu], 0))
    wq_d, s_d = qpc(wd)
    xq, sx = orc.rmsnorm_quant_fp8(to_np(x), code, 1e-5)
    gu = orc.gemm_fp8(xq, wq_gu, sx, s_gu, code)
    aq, sa = orc.swiglu_quant_fp8(gu, code)
    return orc.to_f32(orc.gemm_fp8(aq, wq_d, sa, s_d, code), code)


def test_block_matches_oracle_pipeline():
    T, H, I = 48, 256, 512
    x = randn((T, H), torch.bfloat16, 620)
    wg, wu = randn((I, H), torch.bfloat16, 621, 0.05), randn((I, H), torch.bfloat16, 622, 0.05)
    wd = randn((H, I), torch.bfloat16, 623, 0.05)
    mlp = ql.QuantizedMLP(wg, wu, wd)
    y = mlp(x)
    want = _oracle_mlp(x, wg, wu, wd, orc.BF16)
    assert_close_rel(float_values(y), want, 1e-2, "mlp block")
    # and close to the unquantized block (fp8 noise only)
    xf = x.double()
    r = xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + 1e-5)
    ref = (torch.nn.functional.silu(r @ wg.double().T) * (r @ wu.double().T)) @ wd.double().T
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
