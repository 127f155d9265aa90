"""Parity of the CUDA quantize / dequantize / amax kernels with the CPU oracle, through the C ABI.
Quantized outputs must be bit-exact; dequantized outputs are bit-exact too (one f32 multiply and
one rounding on both sides), which is stricter than the <= 1e-5 relative bound asked for f32."""
import numpy as np
import pytest
import torch

import oracle as orc
import qlinear as ql
from helpers import QL_OF_CODE, code_of, randn, to_np

pytestmark = pytest.mark.gpu

FLOATS = [torch.float32, torch.float16, torch.bfloat16]
QUANTS = [orc.I8, orc.F8E4M3, orc.I4]


def _oracle_q(x, s, qcode, mode, axis, fp8_mode=0):
    return orc.quantize(to_np(x), code_of(x), to_np(s), code_of(s), qcode, mode, axis, fp8_mode)


def _check_q(x, s, qcode, mode, axis=None, fp8_mode="direct"):
    q = ql.quantize(x, s, QL_OF_CODE[qcode], axis, fp8_mode=fp8_mode)
    want = _oracle_q(x, s, qcode, mode, axis, ql._lib.FP8_MODES[fp8_mode])
    got = to_np(q)
    assert got.shape == want.shape
    assert np.array_equal(got, want), f"{(got != want).sum()} of {got.size} differ"
    return q


def _check_dq(q, s, out_torch, mode, axis=None):
    out_dt = ql.dtypes.from_torch(out_torch)
    y = ql.dequantize(q, s, out_dt, axis)
    want = orc.dequantize(to_np(q), code_of(q), to_np(s), code_of(s), out_dt.code, tuple(q.shape), mode, axis)
    assert np.array_equal(to_np(y).view(np.uint8), want.view(np.uint8))
    return y


@pytest.mark.parametrize("in_dtype", FLOATS)
@pytest.mark.parametrize("qcode", QUANTS)
def test_per_tensor_round_trip(in_dtype, qcode):
    x = randn((37, 129), in_dtype, 11)  # ragged: exercises the scalar tail
    amax = x.float().abs().max()
    s = (amax / orc.MAXBOUND[qcode]).to(in_dtype)
    q = _check_q(x, s, qcode, orc.PER_TENSOR)
    _check_dq(q, s, in_dtype, orc.PER_TENSOR)


@pytest.mark.parametrize("in_dtype", FLOATS)
@pytest.mark.parametrize("qcode", QUANTS)
@pytest.mark.parametrize("shape,axis", [((64, 256), 0), ((64, 256), 1), ((3, 16, 64), 1), ((5, 7, 9), 2), ((5, 7, 9), 0)])
def test_per_channel(in_dtype, qcode, shape, axis):
    x = randn(shape, in_dtype, 12)
    red = [d for d in range(len(shape)) if d != axis]
    s = (x.float().abs().amax(dim=red) / orc.MAXBOUND[qcode]).clamp_min(1e-3).to(in_dtype)
    q = _check_q(x, s, qcode, orc.PER_CHANNEL, axis)
    _check_dq(q, s, in_dtype, orc.PER_CHANNEL, axis)


@pytest.mark.parametrize("in_dtype", FLOATS)
@pytest.mark.parametrize("qcode", [orc.I4, orc.F8E4M3])
@pytest.mark.parametrize("shape,sshape", [((256, 128), (2, 128)), ((64, 512), (64, 4)), ((6, 10), (3, 10)), ((6, 10), (6, 5)), ((8, 8), (8, 8))])
def test_block(in_dtype, qcode, shape, sshape):
    x = randn(shape, in_dtype, 13, std=0.02)
    g = torch.Generator(device="cpu").manual_seed(5)
    s = (torch.rand(sshape, generator=g) * 0.01 + 0.002).to(in_dtype).cuda()
    # the operator layer mirrors Tripy (block-wise is int4 only); fp8 block goes through the C ABI rules
    if qcode == orc.F8E4M3:
        q = torch.empty(shape, dtype=torch.float8_e4m3fn, device="cuda")
        from qlinear._lib import check, lib, make_attrs
        from qlinear.tensor import current_stream, ql_view
        check(lib().ql_quantize(ql_view(x), ql_view(s), ql_view(q), make_attrs(), current_stream(x.device)))
        want = _oracle_q(x, s, qcode, orc.BLOCK, None)
        assert np.array_equal(to_np(q), want)
        y = torch.empty(shape, dtype=in_dtype, device="cuda")
        check(lib().ql_dequantize(ql_view(q), ql_view(s), ql_view(y), make_attrs(), current_stream(x.device)))
        wy = orc.dequantize(to_np(q), qcode, to_np(s), code_of(s), code_of(y), shape, orc.BLOCK)
        assert np.array_equal(to_np(y).view(np.uint8), wy.view(np.uint8))
    else:
        q = _check_q(x, s, qcode, orc.BLOCK)
        _check_dq(q, s, in_dtype, orc.BLOCK)


@pytest.mark.parametrize("mode", ["direct", "via_f16", "stablehlo"])
@pytest.mark.parametrize("in_dtype", FLOATS)
def test_fp8_modes(mode, in_dtype):
    x = randn((128, 320), in_dtype, 14, std=3.0)
    x.view(-1)[:6] = torch.tensor([float("nan"), float("inf"), -float("inf"), 1e30, -1e30, 0.0]).to(in_dtype)
    s = torch.tensor(0.02).to(in_dtype)
    _check_q(x, s, orc.F8E4M3, orc.PER_TENSOR, fp8_mode=mode)


@pytest.mark.parametrize("in_dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("qcode", [orc.I8, orc.I4])
def test_integer_quantize_in_the_input_type(in_dtype, qcode):
    """The StableHLO pattern divides in the input's element type: the quotient is rounded to f16 / bf16 before the
    round to integer, which moves values that sit just off a half.  All 16-bit patterns of a range, three scales,
    per-tensor (vector path) and per-channel on a ragged shape (scalar path)."""
    bits = torch.arange(0, 1 << 16, dtype=torch.int32).to(torch.int16).view(in_dtype)
    x = bits[torch.isfinite(bits.float()) & (bits.float().abs() < 200.0)].cuda()
    differ = 0
    for scale in (1.0009765625, 0.3, 1.75):
        s = torch.tensor(scale).to(in_dtype)
        q = _check_q(x, s, qcode, orc.PER_TENSOR, fp8_mode="stablehlo")
        differ += int((to_np(q) != to_np(ql.quantize(x, s, QL_OF_CODE[qcode]))).sum())
    assert differ > 0   # the two arithmetics are not the same function
    xr = x[: 37 * 129].reshape(37, 129).contiguous()
    sc = (torch.rand(129, generator=torch.Generator().manual_seed(3)) + 0.25).to(in_dtype).cuda()
    _check_q(xr, sc, qcode, orc.PER_CHANNEL, 1, fp8_mode="stablehlo")


@pytest.mark.parametrize("qcode", QUANTS)
@pytest.mark.parametrize("in_dtype", [torch.float16, torch.bfloat16])
def test_every_16_bit_input_over_a_range_of_scales(in_dtype, qcode):
    """The kernels divide by a scale that many values share through its reciprocal and two FMA corrections; the
    result must be the IEEE quotient's.  Every bit pattern of the input type (signed zeros, subnormals, infinities
    and NaNs included) against scales from 1e-30 to 1e30 (the ends take the general division), per tensor and, for
    the chunked kernel, per channel."""
    x = torch.arange(0, 1 << 16, dtype=torch.int32).to(torch.int16).view(in_dtype).cuda()
    for scale in (1e-30, 2.0 ** -41, 2.0 ** -40, 1.1e-5, 0.0123, 1.0 / 3.0, 1.0, 1.0009765625, 3.0, 448.0, 1000.7, 2.0 ** 40, 1e30):
        s = torch.tensor(scale, dtype=torch.float32).to(in_dtype)
        if not torch.isfinite(s) or float(s) == 0.0:
            continue
        _check_q(x, s, qcode, orc.PER_TENSOR)
    xc = x.reshape(64, 1024).contiguous()
    sc = torch.logspace(-12, 12, 64, base=2.0).to(in_dtype).cuda()
    _check_q(xc, sc, qcode, orc.PER_CHANNEL, 0)


def test_f32_inputs_of_every_magnitude_divide_exactly():
    """f32 numerators from the subnormals to the largest finite value, both signs, scales across the guarded range."""
    g = torch.Generator(device="cpu").manual_seed(77)
    bits = torch.randint(0, 2 ** 31 - 1, (1 << 20,), generator=g, dtype=torch.int32)
    bits = bits | (torch.randint(0, 2, (1 << 20,), generator=g, dtype=torch.int32) << 31)
    x = bits.view(torch.float32).cuda()
    for scale in (2.0 ** -45, 2.0 ** -39, 7.3e-4, 0.77, 5.0, 2.0 ** 39, 2.0 ** 45):
        for qcode in QUANTS:
            _check_q(x, torch.tensor(scale), qcode, orc.PER_TENSOR)


def test_fp8_every_tie_and_boundary():
    """All e4m3 rounding boundaries and their f32 neighbours, both signs, scale 1."""
    exps = np.arange(-12, 11)
    ties = ((np.arange(16, 32)[None, :] + 0.5) / 16.0 * (2.0 ** exps)[:, None]).reshape(-1).astype(np.float32)
    grid = (np.arange(16, 32)[None, :] / 16.0 * (2.0 ** exps)[:, None]).reshape(-1).astype(np.float32)
    v = np.concatenate([ties, np.nextafter(ties, np.float32(0)), np.nextafter(ties, np.float32(1e9)), grid,
                        np.array([448, 464, 465, 480, 1e9, 2.0 ** -10, 2.0 ** -9, 0.0], dtype=np.float32)])
    v = np.concatenate([v, -v])
    x = torch.from_numpy(v).cuda()
    for mode in ("direct", "via_f16"):
        _check_q(x, torch.tensor(1.0), orc.F8E4M3, orc.PER_TENSOR, fp8_mode=mode)


def test_int_ties_saturation_and_specials():
    v = np.array([0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 126.5, 127.5, 1e9, -128.5, -129.5, -1e9, np.nan, np.inf, -np.inf,
                  6.5, 7.5, -7.5, -8.5, 0.49999997, 3.5000002], dtype=np.float32)
    x = torch.from_numpy(np.tile(v, 40)).cuda()
    for qcode in (orc.I8, orc.I4):
        q = _check_q(x, torch.tensor(1.0), qcode, orc.PER_TENSOR)
    q8 = to_np(ql.quantize(x, 1.0, ql.int8))[: v.size].tolist()
    assert q8[:15] == [0, 2, 2, 0, -2, -2, 126, 127, 127, -128, -128, -128, 0, 127, -128]


@pytest.mark.parametrize("in_dtype", FLOATS)
@pytest.mark.parametrize("qcode", QUANTS)
def test_fused_round_trip_equals_two_steps(in_dtype, qcode):
    x = randn((63, 1000), in_dtype, 15)
    s = (x.float().abs().max() / orc.MAXBOUND[qcode]).to(in_dtype)
    q, y = ql.quantize_dequantize(x, s, QL_OF_CODE[qcode])
    q2 = ql.quantize(x, s, QL_OF_CODE[qcode])
    y2 = ql.dequantize(q2, s, ql.dtypes.from_torch(in_dtype))
    assert np.array_equal(to_np(q), to_np(q2))
    assert np.array_equal(to_np(y).view(np.uint8), to_np(y2).view(np.uint8))
    want = _oracle_q(x, s, qcode, orc.PER_TENSOR, None)
    assert np.array_equal(to_np(q), want)


def test_unaligned_and_empty_inputs():
    base = randn((4099,), torch.float32, 16)
    x = base[3:]  # 12-byte offset: not 16-byte aligned
    assert x.data_ptr() % 16 != 0
    _check_q(x, torch.tensor(0.03), orc.I8, orc.PER_TENSOR)
    _check_q(x, torch.tensor(0.03), orc.I4, orc.PER_TENSOR)
    e = torch.empty((0, 8), device="cuda")
    assert ql.quantize(e, 1.0, ql.int8).numel() == 0
    assert ql.dequantize(torch.empty((0,), dtype=torch.int8, device="cuda"), 1.0, ql.float32).numel() == 0


def test_known_answers_through_the_c_abi(kat):
    """The reference's own test vectors (tests/golden/reference_kat.json) on the GPU path."""
    TD = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
    QD = {"i8": ql.int8, "f8": ql.float8, "i4": ql.int4}
    for case in kat["quantize"]:
        if case["mode"] == "block":
            continue  # fp8 block mode is covered by test_block (Tripy's layer restricts block to int4)
        for dtn in case["in_dtypes"]:
            x = torch.tensor(case["x"], dtype=torch.float32).reshape(case["shape"]).to(TD[dtn]).cuda()
            s = torch.tensor(case["scale"], dtype=torch.float32).to(TD[dtn])
            q = ql.quantize(x, s, QD[case["q_dtype"]], case.get("axis"))
            if case["q_dtype"] == "i8":
                assert q.reshape(-1).tolist() == case["expect"], case["id"]
            else:
                want = torch.tensor(case["expect_f32"]).to(torch.float8_e4m3fn).float()
                assert torch.equal(q.float().cpu().reshape(-1), want), case["id"]
    for case in kat["dequantize"]:
        if case["mode"] == "block":
            continue
        for dtn in case["out_dtypes"]:
            if "q" in case:
                q = torch.tensor(case["q"], dtype=torch.int8).reshape(case["shape"]).cuda()
            else:
                q = torch.tensor(case["q_f32"]).reshape(case["shape"]).to(torch.float8_e4m3fn).cuda()
            s = torch.tensor(case["scale"], dtype=torch.float32).to(TD[dtn])
            y = ql.dequantize(q, s, ql.dtypes.from_torch(TD[dtn]), case.get("axis"))
            want = torch.tensor(case["expect"]).reshape(case["shape"])
            assert torch.allclose(y.float().cpu(), want, rtol={"f32": 1e-5, "f16": 1e-3, "bf16": 8e-3}[dtn]), case["id"]
    c = kat["int4_qdq_identity"]
    for dtn in c["dtypes"]:
        x = torch.full(c["shape"], c["value"], dtype=TD[dtn], device="cuda")
        for case in c["cases"]:
            if case["mode"] == "block":
                s, dim = torch.ones(case["scale_shape"], dtype=TD[dtn]), None
            elif case["mode"] == "pt":
                s, dim = torch.ones((), dtype=TD[dtn]), None
            else:
                s, dim = torch.ones(c["shape"][case["axis"]], dtype=TD[dtn]), case["axis"]
            q = ql.quantize(x, s, ql.int4, dim)
            assert set(q.packed.tolist()) == {0x11}
            assert torch.equal(ql.dequantize(q, s, ql.dtypes.from_torch(TD[dtn]), dim), x)
    p = kat["int4_packing"]
    q = ql.quantize(torch.tensor(p["values"], dtype=torch.float32, device="cuda"), 1.0, ql.int4)
    assert q.packed.tolist() == [p["packed_byte"]]


@pytest.mark.parametrize("in_dtype", FLOATS)
def test_amax_scales(in_dtype):
    x = randn((96, 640), in_dtype, 17)
    cases = [
        (dict(), orc.PER_TENSOR, None, None),
        (dict(dim=0), orc.PER_CHANNEL, 0, None),
        (dict(dim=1), orc.PER_CHANNEL, 1, None),
        (dict(block=(1, 128)), orc.BLOCK, None, (96, 5)),
        (dict(block=(0, 32)), orc.BLOCK, None, (3, 640)),
    ]
    for kw, mode, axis, sshape in cases:
        for qd, mb in ((ql.int8, 127.0), (ql.float8, 448.0), (ql.int4, 7.0)):
            s = ql.amax_scale(x, qd, **kw)
            am = orc.amax(to_np(x), code_of(x), mode, axis, sshape)
            want = orc.scale_from_amax(am, mb, code_of(x))
            assert np.array_equal(to_np(s).reshape(-1).view(np.uint8), want.reshape(-1).view(np.uint8)), (kw, qd)
    x3 = randn((4, 6, 50), in_dtype, 18)
    s = ql.amax_scale(x3, ql.int8, dim=1)
    am = orc.amax(to_np(x3), code_of(x3), orc.PER_CHANNEL, 1)
    assert np.array_equal(to_np(s).reshape(-1).view(np.uint8), orc.scale_from_amax(am, 127.0, code_of(x3)).reshape(-1).view(np.uint8))


def test_config1_full_size_per_tensor_int8():
    """Benchmark config 1: x f32 [4096,4096] ~ N(0,1), scale = max|x| / 127; q and y bit-exact."""
    x = randn((4096, 4096), torch.float32, 1001)
    s = ql.amax_scale(x, ql.int8)
    assert float(s) == float(np.float32(np.abs(to_np(x)).max()) / np.float32(127.0))
    q, y = ql.quantize_dequantize(x, s, ql.int8)
    want_q = _oracle_q(x, s, orc.I8, orc.PER_TENSOR, None)
    assert np.array_equal(to_np(q), want_q)
    want_y = orc.dequantize(want_q, orc.I8, to_np(s), orc.F32, orc.F32, (4096, 4096), orc.PER_TENSOR)
    assert np.array_equal(to_np(y), want_y)
    # size-independent properties: idempotence of Q on its own output, and |x - y| <= scale / 2
    q2 = ql.quantize(y, s, ql.int8)
    assert torch.equal(q2, q)
    assert float((x - y).abs().max()) <= float(s) * 0.5 * (1 + 1e-5)


def test_config2_and_3_weight_quantization_full_size():
    """Weights of configs 2 and 3: per-channel int8 of f16 [11008,4096]; block-128 int4 of f16 [4096,4096]."""
    w = randn((11008, 4096), torch.float16, 1002, std=0.02)
    s = ql.amax_scale(w, ql.int8, dim=0)
    q = ql.quantize(w, s, ql.int8, 0)
    want = _oracle_q(w, s, orc.I8, orc.PER_CHANNEL, 0)
    assert np.array_equal(to_np(q), want)
    assert int(q.abs().max()) == 127  # every row's largest magnitude lands on +-127 (or 126 after f16 scale rounding)
    w3 = randn((4096, 4096), torch.float16, 1003, std=0.02)
    s3 = ql.amax_scale(w3, ql.int4, block=(1, 128))
    assert tuple(s3.shape) == (4096, 32)
    q3 = ql.quantize(w3, s3, ql.int4)
    want3 = _oracle_q(w3, s3, orc.I4, orc.BLOCK, None)
    assert np.array_equal(to_np(q3), want3)
    v = q3.unpack()
    assert int(v.max()) == 7 and int(v.min()) >= -8


@pytest.mark.parametrize("qdt", [ql.float8, ql.int4])
def test_cast_into_and_out_of_quantized_types(qdt):
    """Tripy's cast: quantize / dequantize per tensor with scale 1.0
    (tripy/nvtripy/frontend/ops/cast.py:48-52, tests/integration/test_cast.py:64-74)."""
    x = torch.tensor([-1.0, 0.0, 0.0, 1.0, 2.5, -3.5, 6.0, 100.0], device="cuda")
    q = ql.cast(x, qdt)
    want = ql.quantize(x, 1.0, qdt)
    assert np.array_equal(to_np(q), to_np(want))
    back = ql.cast(q, ql.float32)
    assert torch.equal(back, ql.dequantize(q, 1.0, ql.float32))
    assert ql.cast(q, ql.bool).tolist() == [True, False, False, True, True, True, True, True]
    assert ql.cast(x.to(torch.float16), qdt).shape == q.shape   # 16-bit inputs go through float32, as in Tripy
