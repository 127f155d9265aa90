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
    for name in ("ql_quantize", "ql_dequantize", "ql_linear_w8a16", "ql_linear_w4a16", "ql_gemm_fp8", "ql_gemm_i8"):
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
