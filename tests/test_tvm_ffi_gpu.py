"""The TVM-FFI plug-in library (the reference's `executor.call_plugin` boundary): functions are
resolved by name from the shared object and called with tensors, outputs passed as arguments."""
import os

import numpy as np
import pytest
import torch

from conftest import ROOT

import oracle as orc
import qlinear as ql

PLUGIN = os.path.join(ROOT, "tensorrt-incubator_b200", "lib", "libqlinear_b200_tvmffi.so")
tvm_ffi = pytest.importorskip("tvm_ffi")


def test_plugin_exports_the_expected_functions():
    if not os.path.exists(PLUGIN):
        pytest.skip("plug-in not built (tvm_ffi headers missing at build time)")
    import ctypes
    L = ctypes.CDLL(PLUGIN)
    for name in ("ql_quantize", "ql_dequantize", "ql_linear_w8a16", "ql_linear_w4a16", "ql_gemm_fp8", "ql_gemm_i8", "ql_gemm_16",
                 "ql_linear", "ql_matmul", "ql_dynamic_quantize", "ql_dequantize_nvfp4", "ql_gemm_nvfp4", "ql_rmsnorm_quant_fp8",
                 "ql_gemm_fp8_swiglu", "ql_quantize_rows_fp8"):
        assert hasattr(L, "__tvm_ffi_" + name)


@pytest.mark.gpu
def test_quantize_and_linear_through_tvm_ffi():
    if not os.path.exists(PLUGIN):
        pytest.skip("plug-in not built")
    mod = tvm_ffi.load_module(PLUGIN)
    g = torch.Generator(device="cpu").manual_seed(21)
    x = torch.randn((32, 256), generator=g).cuda()
    s = (x.abs().max() / 127).reshape(())
    q = torch.empty((32, 256), dtype=torch.int8, device="cuda")
    mod.ql_quantize(x, s, q)
    torch.cuda.synchronize()
    want = orc.quantize(x.cpu().numpy(), orc.F32, s.cpu().numpy(), orc.F32, orc.I8)
    assert np.array_equal(q.cpu().numpy(), want)
    y = torch.empty_like(x)
    mod.ql_dequantize(q, s, y)
    torch.cuda.synchronize()
    assert torch.equal(y, ql.dequantize(q, s, ql.float32))

    # per-channel weights, then the weight-only linear
    w = (torch.randn((64, 128), generator=g) * 0.02).to(torch.float16).cuda()
    ws = ql.amax_scale(w, ql.int8, dim=0)
    wq = torch.empty((64, 128), dtype=torch.int8, device="cuda")
    mod.ql_quantize(w, ws, wq, 0)
    xa = torch.randn((4, 128), generator=g).to(torch.float16).cuda()
    out = torch.empty((4, 64), dtype=torch.float16, device="cuda")
    mod.ql_linear_w8a16(xa, wq, ws, out)
    torch.cuda.synchronize()
    assert torch.equal(wq, ql.quantize(w, ws, ql.int8, 0))
    assert torch.equal(out, ql.linear_w8a16(xa, wq, ws))

    # argument errors surface as exceptions, not aborts
    with pytest.raises(Exception, match="axis value must be provided"):
        mod.ql_quantize(w, ws, wq)


@pytest.mark.gpu
def test_linear_matmul_nvfp4_and_mlp_stages_through_tvm_ffi():
    """The entries added for tp.Linear / tp.matmul, NVFP4 and the MLP block's stages: same results as the C ABI
    reached through the operator layer (which the parity tests hold against the oracle)."""
    if not os.path.exists(PLUGIN):
        pytest.skip("plug-in not built")
    mod = tvm_ffi.load_module(PLUGIN)
    g = torch.Generator(device="cpu").manual_seed(22)
    # float32 linear with bias, K = 4 (the shape of the reference's Linear known answers), and a plain matmul
    x = torch.randn((2, 4), generator=g).cuda()
    w = torch.randn((3, 4), generator=g).cuda()
    b = torch.randn((3,), generator=g).cuda()
    y = torch.empty((2, 3), device="cuda")
    mod.ql_linear(x, w, None, None, b, y)
    c = torch.empty((2, 2), device="cuda")
    mod.ql_matmul(x, x.T.contiguous(), c)
    torch.cuda.synchronize()
    assert torch.equal(y, ql.linear(x, w, bias=b)) and torch.equal(c, ql.matmul(x, x.T.contiguous()))
    # NVFP4: quantize both operands, multiply, and dequantize one of them
    a = torch.randn((128, 256), generator=g).to(torch.bfloat16).cuda()
    bw = torch.randn((64, 256), generator=g).to(torch.bfloat16).cuda()
    one = torch.ones((), device="cuda")
    qa, sa = torch.empty((128, 128), dtype=torch.uint8, device="cuda"), torch.empty((128, 16), dtype=torch.uint8, device="cuda")   # e4m3 bits
    qb, sb = torch.empty((64, 128), dtype=torch.uint8, device="cuda"), torch.empty((64, 16), dtype=torch.uint8, device="cuda")
    mod.ql_dynamic_quantize(a, one, qa, sa)
    mod.ql_dynamic_quantize(bw, one, qb, sb, -1, 16)
    out = torch.empty((128, 64), dtype=torch.bfloat16, device="cuda")
    mod.ql_gemm_nvfp4(qa, sa, None, qb, sb, None, out)
    back = torch.empty((128, 256), dtype=torch.bfloat16, device="cuda")
    mod.ql_dequantize_nvfp4(qa, sa, one, back)
    torch.cuda.synchronize()
    fa, fsa = ql.dynamic_quantize(a, one)
    fb, fsb = ql.dynamic_quantize(bw, one)
    assert torch.equal(qa.reshape(-1), fa.packed.reshape(-1)) and torch.equal(sa, fsa.view(torch.uint8))
    assert torch.equal(out, ql.gemm_nvfp4(fa, fsa, fb, fsb, out_dtype=ql.bfloat16))
    assert torch.equal(back, ql.dequantize_nvfp4(fa, fsa, one, ql.bfloat16))
    # the MLP block's stages
    h = torch.randn((64, 512), generator=g).to(torch.bfloat16).cuda()
    xq, sx = torch.empty((64, 512), dtype=torch.uint8, device="cuda"), torch.empty(64, device="cuda")
    mod.ql_rmsnorm_quant_fp8(h, 1e-5, xq, sx)
    wq = ql.interleave_gate_up((torch.randn((128, 512), generator=g) * 0.1).cuda(), (torch.randn((128, 512), generator=g) * 0.1).cuda()).to(torch.float8_e4m3fn)
    sw = torch.full((256,), 0.5, device="cuda")
    act, amax = torch.empty((64, 128), dtype=torch.bfloat16, device="cuda"), torch.zeros(64, device="cuda")
    mod.ql_gemm_fp8_swiglu(xq, wq.view(torch.uint8), sx, sw, act, amax)
    aq, sa2 = torch.empty((64, 128), dtype=torch.uint8, device="cuda"), torch.empty(64, device="cuda")
    mod.ql_quantize_rows_fp8(act, amax, aq, sa2)
    torch.cuda.synchronize()
    wxq, wsx = ql.rmsnorm_quant_fp8(h, 1e-5)
    assert torch.equal(xq, wxq.view(torch.uint8)) and torch.equal(sx, wsx)
    wact, wamax = torch.empty_like(act), torch.zeros_like(amax)
    ql.gemm_fp8_swiglu(wxq, wq, wsx, sw, wact, wamax)
    waq, wsa = ql.quantize_rows_fp8(wact, wamax)
    assert torch.equal(act, wact) and torch.equal(amax, wamax) and torch.equal(aq, waq.view(torch.uint8)) and torch.equal(sa2, wsa)
    with pytest.raises(Exception, match="expected"):
        mod.ql_matmul(x, x)
