"""Weight-only linear kernels against the oracle (f64 accumulation), through the C ABI.
Tolerance: relative 1e-2 of max(|reference|, rms(reference)), the benchmark's bound for
16-bit outputs; the observed error is the output rounding (2^-9 bf16, 2^-11 f16)."""
import numpy as np
import pytest
import torch

import oracle as orc
import qlinear as ql
from helpers import assert_close_rel, code_of, float_values, randn, to_np

pytestmark = pytest.mark.gpu


def _w8_case(M, N, K, xdtype, seed):
    w = randn((N, K), torch.float16, seed, std=0.02)
    s = ql.amax_scale(w, ql.int8, dim=0)
    q = ql.quantize(w, s, ql.int8, 0)
    x = randn((M, K), xdtype, seed + 1)
    return x, q, s


@pytest.mark.parametrize("xdtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K", [(1, 64, 256), (3, 48, 128), (8, 40, 512), (16, 64, 1024), (17, 33, 64), (32, 128, 2048), (45, 16, 192)])
def test_w8a16_matches_oracle(xdtype, M, N, K):
    x, q, s = _w8_case(M, N, K, xdtype, 200 + M)
    y = ql.linear_w8a16(x, q, s)
    want = orc.linear_w8(to_np(x), code_of(x), to_np(q), to_np(s), code_of(s), orc.F32, acc64=True)
    assert_close_rel(float_values(y), want, 1e-2, f"w8a16 {M}x{N}x{K}")
    # far tighter than the contract: only the final rounding to 16 bits separates the two
    ulp = 2.0 ** -8 if xdtype == torch.bfloat16 else 2.0 ** -10
    assert_close_rel(float_values(y), want, ulp, "w8a16 tight")


@pytest.mark.parametrize("xdtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M,N,K,B", [(1, 32, 256, 128), (8, 64, 512, 128), (5, 24, 384, 128), (32, 48, 1024, 256), (16, 16, 128, 128)])
def test_w4a16_matches_oracle(xdtype, M, N, K, B):
    w = randn((N, K), xdtype, 300 + M, std=0.02)
    s = ql.amax_scale(w, ql.int4, block=(1, B))
    q = ql.quantize(w, s, ql.int4)
    x = randn((M, K), xdtype, 301 + M)
    y = ql.linear_w4a16(x, q, s)
    want = orc.linear_w4(to_np(x), code_of(x), to_np(q), to_np(s), code_of(s), orc.F32, B, acc64=True)
    assert_close_rel(float_values(y), want, 1e-2, f"w4a16 {M}x{N}x{K}")
    ulp = 2.0 ** -8 if xdtype == torch.bfloat16 else 2.0 ** -10
    assert_close_rel(float_values(y), want, ulp, "w4a16 tight")


@pytest.mark.parametrize("xdtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K", [(65, 64, 64), (128, 256, 512), (300, 100, 192), (129, 33, 1024), (512, 1000, 256), (96, 4096, 128)])
def test_w8a16_large_batch_fused_tensor_core_path(xdtype, M, N, K):
    """M > 64 runs the tcgen05 kernel that widens the int8 weights in shared memory."""
    import ctypes
    x, q, s = _w8_case(M, N, K, xdtype, 700 + M)
    y = ql.linear_w8a16(x, q, s)
    code = ctypes.c_int32(0)
    assert ql.lib().ql_gemm_status(ctypes.byref(code)) == 0 and code.value == 0
    want = orc.linear_w8(to_np(x), code_of(x), to_np(q), to_np(s), code_of(s), orc.F32, acc64=True)
    ulp = 2.0 ** -8 if xdtype == torch.bfloat16 else 2.0 ** -10
    assert_close_rel(float_values(y), want, ulp, f"fused w8a16 {M}x{N}x{K}")


def test_w8a16_small_and_large_batch_paths_agree():
    """The same rows through the streaming kernel (M <= 64) and the tensor-core kernel (M > 64)."""
    x, q, s = _w8_case(192, 512, 1024, torch.bfloat16, 710)
    big = ql.linear_w8a16(x, q, s)
    small = torch.cat([ql.linear_w8a16(x[i:i + 64].contiguous(), q, s) for i in range(0, 192, 64)])
    assert_close_rel(float_values(big), float_values(small).astype(np.float64), 2.0 ** -7, "paths agree")


def test_w8a16_equals_dequantize_then_matmul():
    """The fused kernel against the reference composition dequantize -> matmul computed in f64."""
    x, q, s = _w8_case(16, 256, 512, torch.bfloat16, 400)
    y = ql.linear_w8a16(x, q, s)
    wdq = ql.dequantize(q, s.float(), ql.float32, 0)
    want = (x.double() @ wdq.double().T).cpu().numpy()
    assert_close_rel(float_values(y), want, 2.0 ** -8, "vs dq+matmul")


@pytest.mark.parametrize("M", [1, 16, 128])
def test_config2_shapes(M):
    """Config 2 at full N, K for M in {1, 16, 128}; the oracle checks a slice of output channels."""
    x, q, s = _w8_case(M, 11008, 4096, torch.bfloat16, 1002)
    y = ql.linear_w8a16(x, q, s)
    sl = slice(5000, 5064)
    want = orc.linear_w8(to_np(x), code_of(x), to_np(q[sl]), to_np(s[sl]), code_of(s), orc.F32, acc64=True)
    assert_close_rel(float_values(y[:, sl]), want, 2.0 ** -8, f"config 2 M={M}")
    # linearity in x (size-independent property): f(2x) == 2 f(x) exactly, powers of two are exact
    y2 = ql.linear_w8a16(x * 2, q, s)
    assert torch.equal(y2, y * 2)


@pytest.mark.parametrize("xdtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K", [(2048, 11008, 4096), (2200, 9000, 320), (1025, 19000, 64)])
def test_w8a16_compute_bound_single_launch_path(xdtype, M, N, K, monkeypatch):
    """M > 256 with enough tiles: the CTA-pair GEMM that widens the weights ahead of its own tiles, against the
    oracle on slices of rows and channels (first, ragged last chunk, middle) and, bit for bit, against the route that
    widens in a kernel of its own."""
    import ctypes
    x, q, s = _w8_case(M, N, K, xdtype, 1200 + M)
    c0 = ql.lib().ql_launch_count()
    y = ql.linear_w8a16(x, q, s)
    assert ql.lib().ql_launch_count() - c0 == 1
    for _ in range(2):   # the kernel must leave its tile counters ready for the next launch
        y_again = ql.linear_w8a16(x, q, s)
    assert torch.equal(y, y_again)
    code = ctypes.c_int32(0)
    assert ql.lib().ql_gemm_status(ctypes.byref(code)) == 0 and code.value == 0
    ulp = 2.0 ** -8 if xdtype == torch.bfloat16 else 2.0 ** -10
    rows = slice(M - 40, M)
    for sl in (slice(0, 48), slice(N - 40, N), slice(N // 2 - 7, N // 2 + 25)):
        want = orc.linear_w8(to_np(x[rows]), code_of(x), to_np(q[sl]), to_np(s[sl]), code_of(s), orc.F32, acc64=True)
        assert_close_rel(float_values(y[rows, sl]), want, ulp, f"single-launch w8a16 {M}x{N}x{K} channels {sl}")
    monkeypatch.setenv("QL_W8_TWO_KERNELS", "1")
    ql.lib().ql_reload_tuning()   # the tuning variables are read once per process otherwise
    try:
        c0 = ql.lib().ql_launch_count()
        y_two = ql.linear_w8a16(x, q, s)
        assert ql.lib().ql_launch_count() - c0 == 3
        assert torch.equal(y, y_two)
    finally:
        monkeypatch.delenv("QL_W8_TWO_KERNELS")
        ql.lib().ql_reload_tuning()


@pytest.mark.parametrize("M", [1, 8, 32])
def test_config3_shapes(M):
    w = randn((4096, 4096), torch.float16, 1003, std=0.02)
    s = ql.amax_scale(w, ql.int4, block=(1, 128))
    q = ql.quantize(w, s, ql.int4)
    x = randn((M, 4096), torch.float16, 1004)
    y = ql.linear_w4a16(x, q, s)
    sl = slice(1000, 1048)
    qs = ql.Int4Tensor(q.packed.reshape(4096, 2048)[sl].reshape(-1).contiguous(), (48, 4096))
    want = orc.linear_w4(to_np(x), code_of(x), to_np(qs), to_np(s[sl]), code_of(s), orc.F32, 128, acc64=True)
    assert_close_rel(float_values(y[:, sl]), want, 2.0 ** -10, f"config 3 M={M}")


def test_linear_module_mirrors_tripy_linear():
    """tp.Linear with int8 weights, weight_quant_dim 0, no input scale: iota weights, ones input,
    as tripy/tests/integration/test_linear.py:87-110 builds them."""
    lin = ql.Linear(64, 16, bias=False, dtype=ql.float16, quant_dtype=ql.int8, weight_quant_dim=0)
    wt = torch.arange(16 * 64, dtype=torch.float32).reshape(16, 64).to(torch.float16)
    lin.load_state_dict({"weight": wt, "weight_scale": torch.ones(16, dtype=torch.float16)})
    x = torch.ones(2, 64, dtype=torch.float16, device="cuda")
    out = lin(x)
    # weights above 127 saturate, exactly as quantize -> dequantize -> matmul does
    want = x.float() @ wt.float().clamp(-128, 127).cuda().T
    assert torch.allclose(out.float(), want, rtol=1e-3)
