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


@pytest.mark.parametrize("xdtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K", [(128, 11008, 4096), (70, 1000, 2048), (33, 320, 512), (128, 4100, 1024)])
def test_w8a16_one_row_tile_splits_k_over_a_cluster(xdtype, M, N, K, monkeypatch, ksplit=2):
    """M <= 128: a cluster of two CTAs shares a column tile, each takes half of K and the partial sums are
    added through distributed shared memory in rank order.  Every channel against the oracle (ragged last tile
    included), the status word clean, and the result identical from call to call (the order of the sum is fixed)."""
    import ctypes
    x, q, s = _w8_case(M, N, K, xdtype, 760 + M + ksplit)
    monkeypatch.setenv("QL_W8_KSPLIT", str(ksplit))
    ql.lib().ql_reload_tuning()
    try:
        y = torch.full((M, N), float("nan"), dtype=xdtype, device="cuda")
        y.copy_(ql.linear_w8a16(x, q, s))
        again = ql.linear_w8a16(x, q, s)
    finally:
        monkeypatch.delenv("QL_W8_KSPLIT")
        ql.lib().ql_reload_tuning()
    code = ctypes.c_int32(0)
    assert ql.lib().ql_gemm_status(ctypes.byref(code)) == 0 and code.value == 0
    assert torch.equal(y, again)
    cols = slice(0, N) if N <= 1000 else slice(N - 700, N)
    want = orc.linear_w8(to_np(x), code_of(x), to_np(q[cols]), to_np(s[cols]), code_of(s), orc.F32, acc64=True)
    ulp = 2.0 ** -8 if xdtype == torch.bfloat16 else 2.0 ** -10
    assert_close_rel(float_values(y[:, cols]), want, ulp, f"k split {ksplit}: {M}x{N}x{K}")
    if N > 1000:   # the other channels against the unsplit kernel, which the oracle covers elsewhere
        monkeypatch.setenv("QL_W8_KSPLIT", "1")
        ql.lib().ql_reload_tuning()
        try:
            whole = ql.linear_w8a16(x, q, s)
        finally:
            monkeypatch.delenv("QL_W8_KSPLIT")
            ql.lib().ql_reload_tuning()
        assert_close_rel(float_values(y), float_values(whole).astype(np.float64), 2 * ulp, "split against unsplit")


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


def _w8_layer(N, K, seed):
    w = randn((N, K), torch.float16, seed, std=0.02)
    s = ql.amax_scale(w, ql.int8, dim=0)
    return ql.quantize(w, s, ql.int8, 0), s


def test_w8a16_scratch_is_per_call_graph_replay_after_a_larger_layer():
    """The compute-bound route (more than 256 rows) widens the weights into scratch taken per call from the
    stream-ordered allocator.  A graph captured for a small layer must still be right after a larger layer has run
    (nothing it refers to may have been freed or moved), and again after the large layer's own graph."""
    q1, s1 = _w8_layer(512, 256, 1301)
    q2, s2 = _w8_layer(4096, 2048, 1302)
    x1, x2 = randn((320, 256), torch.bfloat16, 1303), randn((1024, 2048), torch.bfloat16, 1304)
    want1, want2 = ql.linear_w8a16(x1, q1, s1).clone(), ql.linear_w8a16(x2, q2, s2).clone()
    y1 = torch.empty_like(want1)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        ql.linear_w8a16(x1, q1, s1, out=y1)   # warm-up on the capture stream
    torch.cuda.current_stream().wait_stream(side)
    g1 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g1):
        ql.linear_w8a16(x1, q1, s1, out=y1)
    y1.zero_()
    g1.replay()
    torch.cuda.synchronize()
    assert torch.equal(y1, want1)
    for _ in range(2):
        assert torch.equal(ql.linear_w8a16(x2, q2, s2), want2)   # the larger layer, eagerly
        y1.zero_()
        g1.replay()
        torch.cuda.synchronize()
        assert torch.equal(y1, want1)
    assert ql.lib().ql_gemm_status(None) == 0


def test_w8a16_calls_on_two_streams_do_not_share_scratch():
    q1, s1 = _w8_layer(2048, 1024, 1311)
    q2, s2 = _w8_layer(1024, 2048, 1312)
    x1, x2 = randn((768, 1024), torch.bfloat16, 1313), randn((640, 2048), torch.float16, 1314)
    want1, want2 = ql.linear_w8a16(x1, q1, s1).clone(), ql.linear_w8a16(x2, q2, s2).clone()
    torch.cuda.synchronize()
    a, b = torch.cuda.Stream(), torch.cuda.Stream()
    outs = []
    for i in range(6):
        with torch.cuda.stream(a):
            ya = ql.linear_w8a16(x1, q1, s1)
        with torch.cuda.stream(b):
            yb = ql.linear_w8a16(x2, q2, s2)
        outs.append((ya, yb))
    torch.cuda.synchronize()
    for ya, yb in outs:
        assert torch.equal(ya, want1) and torch.equal(yb, want2)
    assert ql.lib().ql_gemm_status(None) == 0


def test_weights_constant_flag_gives_the_same_result():
    """QL_WEIGHTS_CONSTANT only changes when the kernel may start; back-to-back launches that overlap must each still
    see their own, complete activations."""
    q, s = _w8_layer(4096, 1024, 1321)
    w4 = randn((4096, 1024), torch.float16, 1322, std=0.02)
    s4 = ql.amax_scale(w4, ql.int4, block=(1, 128))
    q4 = ql.quantize(w4, s4, ql.int4)
    torch.cuda.synchronize()
    for m in (1, 8, 24):
        xs = [randn((m, 1024), torch.float16, 1330 + i) for i in range(4)]
        plain = [ql.linear_w8a16(x, q, s) for x in xs]
        plain4 = [ql.linear_w4a16(x, q4, s4) for x in xs]
        torch.cuda.synchronize()
        # a chain: each launch's input is rewritten by a kernel right before it
        buf = torch.empty_like(xs[0])
        got, got4 = [], []
        for x in xs:
            buf.copy_(x)
            got.append(ql.linear_w8a16(buf, q, s, weights_constant=True).clone())
            buf.copy_(x)
            got4.append(ql.linear_w4a16(buf, q4, s4, weights_constant=True).clone())
        torch.cuda.synchronize()
        for a_, b_ in zip(plain + plain4, got + got4):
            assert torch.equal(a_, b_)
