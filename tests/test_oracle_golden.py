"""The CPU oracle against the known-answer vectors of the reference's own tests
(tests/golden/reference_kat.json, each entry citing the reference test it was read from)."""
import math

import numpy as np
import pytest

from linear_cases import iota as _iota, linear_cases as _linear_cases

CODE = {"f32": 0, "f16": 1, "bf16": 2, "i8": 3, "i4": 4, "f8": 5}
MODE = {"pt": 0, "pc": 1, "block": 2}


def _scale_array(orc, case, dt):
    s = np.array(case["scale"], dtype=np.float32)
    if "scale_shape" in case:
        s = s.reshape(case["scale_shape"])
    return orc.from_f32(s, CODE[dt])


def _f8_decode(orc, bits):
    L = orc.lib()
    return np.array([L.orc_f8e4m3_to_f32(int(b)) for b in bits.reshape(-1)], dtype=np.float32)


def _f8_encode(orc, vals):
    L = orc.lib()
    return np.array([L.orc_f32_to_f8e4m3(float(v)) for v in vals], dtype=np.uint8)


def test_quantize_known_answers(orc, kat):
    for case in kat["quantize"]:
        for dt in case["in_dtypes"]:
            x = orc.from_f32(np.array(case["x"], dtype=np.float32).reshape(case["shape"]), CODE[dt])
            s = _scale_array(orc, case, dt)
            q = orc.quantize(x, CODE[dt], s, CODE[dt], CODE[case["q_dtype"]], MODE[case["mode"]], case.get("axis"))
            if case["q_dtype"] == "i8":
                assert q.reshape(-1).tolist() == case["expect"], (case["id"], dt)
            else:
                # the reference tests compare after casting the expectation to e4m3
                want = _f8_decode(orc, _f8_encode(orc, case["expect_f32"]))
                got = _f8_decode(orc, q)
                assert np.array_equal(got, want), (case["id"], dt)


def test_dequantize_known_answers(orc, kat):
    for case in kat["dequantize"]:
        for dt in case["out_dtypes"]:
            if "q" in case:
                q = np.array(case["q"], dtype=np.int8).reshape(case["shape"])
            else:
                q = _f8_encode(orc, case["q_f32"]).reshape(case["shape"])
            s = _scale_array(orc, case, dt)
            y = orc.dequantize(q, CODE[case["q_dtype"]], s, CODE[dt], CODE[dt], case["shape"], MODE[case["mode"]], case.get("axis"))
            got = orc.to_f32(y, CODE[dt]).reshape(-1)
            want = np.array(case["expect"], dtype=np.float32)
            if case.get("allclose") or dt != "f32":
                # torch.allclose defaults of the reference tests, widened to the output type's ulp
                rtol = {"f32": 1e-5, "f16": 1e-3, "bf16": 8e-3}[dt]
                assert np.allclose(got, want, rtol=rtol, atol=1e-8), (case["id"], dt, got)
            else:
                assert np.array_equal(got, want), (case["id"], dt, got)


def test_fp8_constants(orc, kat):
    c = kat["fp8_constants"]
    bits = _f8_encode(orc, c["f32"])
    y = orc.dequantize(bits, CODE["f8"], np.array(1.0, dtype=np.float32), 0, 0, [4], 0)
    assert (y * 2).tolist() == c["dequantized_times_2"]


def test_int4_round_trip_identity(orc, kat):
    c = kat["int4_qdq_identity"]
    for dt in c["dtypes"]:
        x = orc.from_f32(np.full(c["shape"], c["value"], dtype=np.float32), CODE[dt])
        for case in c["cases"]:
            if case["mode"] == "block":
                s = orc.from_f32(np.ones(case["scale_shape"], dtype=np.float32), CODE[dt])
            elif case["mode"] == "pt":
                s = orc.from_f32(np.ones((), dtype=np.float32), CODE[dt])
            else:
                s = orc.from_f32(np.ones(c["shape"][case["axis"]], dtype=np.float32), CODE[dt])
            q = orc.quantize(x, CODE[dt], s, CODE[dt], CODE["i4"], MODE[case["mode"]], case.get("axis"))
            assert q.dtype == np.uint8 and q.size == 8 and set(q.tolist()) == {0x11}
            y = orc.dequantize(q, CODE["i4"], s, CODE[dt], CODE[dt], c["shape"], MODE[case["mode"]], case.get("axis"))
            assert np.array_equal(y, x), (dt, case)


def test_int4_dequantize_then_matmul(orc, kat):
    for case in kat["int4_dq_matmul"]["cases"]:
        vals = np.array(case["lhs_i4"], dtype=np.int8)
        packed = np.zeros(2, dtype=np.uint8)
        for i, v in enumerate(vals):
            packed[i // 2] |= (int(v) & 0xF) << (4 * (i % 2))
        lhs = orc.dequantize(packed, CODE["i4"], np.array(case["scale"], dtype=np.float32), 0, 0, [2, 2], 0)
        out = lhs @ np.array(case["rhs"], dtype=np.float32).reshape(2, 2)
        assert out.reshape(-1).tolist() == case["expect"]
        # the same product through the weight-only linear entry of the oracle: Y = X . dq(W)^T
        X = np.array(case["rhs"], dtype=np.float32).reshape(2, 2).T.copy()
        Y = orc.linear_w4(X, 0, packed, np.full((2, 1), case["scale"], dtype=np.float32), 0, 0, block=2)
        assert np.array_equal(Y.T, out)


def test_int4_packing_low_nibble_first(orc, kat):
    c = kat["int4_packing"]
    x = np.array(c["values"], dtype=np.float32)
    q = orc.quantize(x, 0, np.array(1.0, dtype=np.float32), 0, CODE["i4"], 0)
    assert q.tolist() == [c["packed_byte"]]
    assert orc.unpack_i4(q, 2).tolist() == c["values"]


def test_f8_type_known_answers(orc, kat):
    L = orc.lib()
    for e in kat["f8_type"]["encode"]:
        v = float(e["f32"])
        b = L.orc_f32_to_f8e4m3(v)
        if "bits" in e:
            assert b == e["bits"], e
        else:
            assert L.orc_f8e4m3_to_f32(b) == e["decodes_to"], e
    for d in kat["f8_type"]["decode"]:
        assert L.orc_f8e4m3_to_f32(d["bits"]) == d["f32"]
    assert math.isnan(L.orc_f8e4m3_to_f32(0x7F))


def test_int4_saturation(orc, kat):
    for e in kat["int4_type"]["saturate"]:
        q = orc.quantize(np.array([e["in"]], dtype=np.float32), 0, np.array(1.0, dtype=np.float32), 0, CODE["i4"], 0)
        assert orc.unpack_i4(q, 1).tolist() == [e["out"]]


def test_round_half_even_and_saturation_follow_the_specification(orc):
    """Not pinned by any reference test: ties go to even, results clamp to the integer range
    (TensorRTOps.td:3138-3153)."""
    x = np.array([0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 126.5, 127.5, 1e9, -128.5, -129.5, -1e9, np.nan], dtype=np.float32)
    q = orc.quantize(x, 0, np.array(1.0, dtype=np.float32), 0, CODE["i8"], 0)
    assert q.tolist() == [0, 2, 2, 0, -2, -2, 126, 127, 127, -128, -128, -128, 0]
    q4 = orc.unpack_i4(orc.quantize(x[:8], 0, np.array(1.0, dtype=np.float32), 0, CODE["i4"], 0), 8)
    assert q4.tolist() == [0, 2, 2, 0, -2, -2, 7, 7]


def test_fp8_modes_differ_where_documented(orc):
    s = np.array(1.0, dtype=np.float32)
    # 0.3 -> e4m3 0.3125 directly; the StableHLO pattern first rounds to an integer (0)
    x = np.array([0.3, 2.4, 500.0], dtype=np.float32)
    d = _f8_decode(orc, orc.quantize(x, 0, s, 0, CODE["f8"], 0, fp8_mode=0))
    h = _f8_decode(orc, orc.quantize(x, 0, s, 0, CODE["f8"], 0, fp8_mode=2))
    assert d.tolist() == [0.3125, 2.5, 448.0]
    assert h.tolist() == [0.0, 2.0, 448.0]
    # double rounding through f16: 1.0625 + 2^-12 is above the e4m3 tie 1.0625 in f32 but
    # lands on the tie after rounding to f16, and the tie goes to even (1.0)
    y = np.array([1.0625 + 2.0 ** -12], dtype=np.float32)
    assert _f8_decode(orc, orc.quantize(y, 0, s, 0, CODE["f8"], 0, fp8_mode=0)).tolist() == [1.125]
    assert _f8_decode(orc, orc.quantize(y, 0, s, 0, CODE["f8"], 0, fp8_mode=1)).tolist() == [1.0]


def test_integer_quantize_in_the_input_type_against_numpy_half_arithmetic(orc):
    """The StableHLO pattern (divide, round_nearest_even, clamp, convert, all on f16 tensors:
    compiler/test/Dialect/StablehloExt/raise-qdq-per-tensor-quantize.mlir) restated with numpy's float16 operators,
    which round every result to f16; the operator's own f32 division differs from it on a few inputs."""
    x = np.arange(0, 1 << 16, dtype=np.uint16).view(np.float16)
    x = x[np.isfinite(x) & (np.abs(x.astype(np.float32)) < 200.0)]
    differ = 0
    for scale in (1.0009765625, 0.3, 1.75):
        s = np.array(scale, dtype=np.float16)
        want = np.clip(np.rint(x / s), np.float16(-128), np.float16(127)).astype(np.int8)
        got = orc.quantize(x, CODE["f16"], s, CODE["f16"], CODE["i8"], 0, fp8_mode=2)
        assert np.array_equal(got, want)
        differ += int((orc.quantize(x, CODE["f16"], s, CODE["f16"], CODE["i8"], 0) != want).sum())
    assert differ > 0


def test_nvfp4_dynamic_quantize_known_answer(orc, kat):
    """The reference's only NVFP4 execution test: quantize to e2m1 with e4m3 block-16 scales, dequantize back."""
    case = kat["nvfp4_dynamic_quantize"]
    x = np.array(case["input"], dtype=np.float32)
    q, s = orc.dynamic_quantize_nvfp4(x, orc.F32, case["double_quant_scale"])
    assert q.shape == (2, 16) and s.shape == (2, 2)
    y = orc.dequantize_nvfp4(q, s, case["double_quant_scale"], orc.F32)
    assert np.array_equal(y, np.array(case["expected"], dtype=np.float32))


def test_e2m1_rounding_is_nearest_even_and_saturating(orc):
    L = orc.lib()
    values = [L.orc_f4e2m1_to_f32(i) for i in range(16)]
    assert values[:8] == [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0] and values[9] == -0.5 and values[15] == -6.0
    # ties go to the code with an even mantissa: 0.25 -> 0, 0.75 -> 1, 1.25 -> 1, 1.75 -> 2, 2.5 -> 2, 3.5 -> 4, 5 -> 4
    for x, want in [(0.25, 0.0), (0.75, 1.0), (1.25, 1.0), (1.75, 2.0), (2.5, 2.0), (3.5, 4.0), (5.0, 4.0), (5.01, 6.0), (1e9, 6.0), (-7.0, -6.0), (0.26, 0.5)]:
        assert L.orc_f4e2m1_to_f32(L.orc_f32_to_f4e2m1(x)) == want, x


def test_linear_module_known_answers(orc, kat):
    """tripy/tests/integration/test_linear.py: float Linear, the twelve int8 / float8 combinations (two rejected)
    and the four int4 weight-only modes, through the oracle's op-by-op restatement of Linear.forward."""
    seen = 0
    for cid, kw, want in _linear_cases(kat):
        if want is None:
            with pytest.raises(ValueError, match=kat["linear_module"]["quant"]["rejected"]["message"]):
                orc.linear_module(**kw)
        else:
            assert np.array_equal(orc.linear_module(**kw), want), cid
        seen += 1
    assert seen == 1 + 12 + 4


def test_matmul_rank_rules(orc, kat):
    for case in kat["matmul_doc_examples"]["cases"]:
        a, b = _iota(case["a_shape"], case["a_iota_dim"]), _iota(case["b_shape"], case["b_iota_dim"])
        got = orc.matmul(a, b, CODE["f32"])
        assert got.shape == (a @ b).shape and np.array_equal(got, a @ b), case
    # the int4 dequantize -> matrix_multiply answers, through the same matmul
    for case in kat["int4_dq_matmul"]["cases"]:
        vals = np.array(case["lhs_i4"], dtype=np.int8)
        packed = np.zeros(2, dtype=np.uint8)
        for i, v in enumerate(vals):
            packed[i // 2] |= (int(v) & 0xF) << (4 * (i % 2))
        lhs = orc.dequantize(packed, CODE["i4"], np.array(case["scale"], dtype=np.float32), 0, 0, [2, 2], 0)
        out = orc.matmul(lhs, np.array(case["rhs"], dtype=np.float32).reshape(2, 2), CODE["f32"])
        assert out.reshape(-1).tolist() == case["expect"]
