"""Argument contract of the operator layer, with the messages Tripy's tests pin
(tripy/tests/frontend/ops/test_quantize.py:24-84, test_dequantize.py, and
tripy/tests/integration/test_linear.py:96-102)."""
import pytest
import torch

import qlinear as ql


def test_quantize_rejects_bad_input_dtype():
    with pytest.raises(ql.QuantizeError, match="Input does not have a valid dtype in quantize op"):
        ql.quantize(torch.ones(2, dtype=torch.int32), 1.0, ql.int8)


def test_quantize_rejects_bad_target_dtype():
    with pytest.raises(ql.QuantizeError, match="Unsupported data type in quantize op"):
        ql.quantize(torch.ones(2), 1.0, ql.float16)


def test_per_channel_needs_1d_scale():
    with pytest.raises(ql.QuantizeError, match="If dim is given, scale must be a 1-D tensor in per-channel quantize op"):
        ql.quantize(torch.ones(4, 4), torch.ones(4, 4), ql.int8, dim=0)


def test_block_needs_2d_input():
    with pytest.raises(ql.QuantizeError, match="Input must be a 2-D tensor in block-wise quantize op"):
        ql.quantize(torch.ones(4), torch.ones(2, 4), ql.int4)


def test_block_needs_int4():
    with pytest.raises(ql.QuantizeError, match="Unsupported data type in block-wise quantize op"):
        ql.quantize(torch.ones(4, 4), torch.ones(2, 4), ql.int8)


def test_per_tensor_needs_scalar_scale():
    with pytest.raises(ql.QuantizeError, match="Scale must be a scalar tensor in per-tensor quantize op"):
        ql.quantize(torch.ones(4, 4), torch.ones(4), ql.int8)


def test_scale_dtype_must_match():
    with pytest.raises(ql.QuantizeError, match="Scale dtype does not match expected dtype"):
        ql.quantize(torch.ones(4, dtype=torch.float16), torch.ones((), dtype=torch.float32), ql.int8)


def test_dequantize_messages():
    with pytest.raises(ql.QuantizeError, match="Input does not have a valid dtype in dequantize op"):
        ql.dequantize(torch.ones(2), 1.0, ql.float32)
    with pytest.raises(ql.QuantizeError, match="Unsupported data type in dequantize op"):
        ql.dequantize(torch.ones(2, dtype=torch.int8), 1.0, ql.int8)
    with pytest.raises(ql.QuantizeError, match="If dim is given, scale must be a 1-D tensor in per-channel dequantize op"):
        ql.dequantize(torch.ones(2, 2, dtype=torch.int8), torch.ones(2, 2), ql.float32, dim=0)
    with pytest.raises(ql.QuantizeError, match="Scale must be a scalar tensor in per-tensor dequantize op"):
        ql.dequantize(torch.ones(2, 2, dtype=torch.int8), torch.ones(2), ql.float32)


def test_int4_pack_unpack_round_trip():
    v = torch.arange(-8, 8, dtype=torch.int8).reshape(4, 4)
    t = ql.Int4Tensor.pack(v)
    assert t.packed.tolist()[0] == 0x98  # -8 -> 0x8 low nibble, -7 -> 0x9 high nibble
    assert torch.equal(t.unpack(), v)
    odd = ql.Int4Tensor.pack(torch.tensor([1, 2, 3], dtype=torch.int8))
    assert odd.packed.tolist() == [0x21, 0x03]


def test_linear_rejects_input_scale_with_weight_quant_dim_1():
    lin = ql.Linear(4, 2, bias=False, dtype=ql.float32, quant_dtype=ql.int8, weight_quant_dim=1, device="cpu")
    lin.weight_scale = torch.ones(4)
    lin.input_scale = torch.tensor(1.0)
    with pytest.raises(ql.QuantizeError, match="Unsupported quantization parameters for Linear module."):
        lin(torch.ones(1, 4))


def test_cast_refuses_what_tripy_refuses():
    """tripy/nvtripy/frontend/ops/cast.py:32-38."""
    q8 = torch.ones(4, dtype=torch.int8)
    f8 = torch.ones(4).to(torch.float8_e4m3fn)
    i4 = ql.Int4Tensor.pack(torch.ones(4, dtype=torch.int8))
    for x, target in [(f8, ql.int4), (f8, ql.int8), (q8, ql.float8), (i4, ql.float8), (i4, ql.int8), (i4, ql.int64)]:
        with pytest.raises(ql.QuantizeError, match="Unsupported cast"):
            ql.cast(x, target)


def test_cast_between_plain_types_is_an_ordinary_conversion():
    x = torch.tensor([1.0, -2.0, 3.5])
    assert ql.cast(x, ql.float32) is x
    assert ql.cast(x, ql.int32).tolist() == [1, -2, 3]
    assert ql.cast(torch.tensor([0, 5], dtype=torch.int8), ql.float32).tolist() == [0.0, 5.0]
    assert ql.cast(torch.tensor([False, True]), ql.int8).tolist() == [0, 1]


def test_matmul_contract():
    """tripy/nvtripy/frontend/ops/matmul.py:31-34 (one float type for both operands) and :98-102 (no scalars)."""
    x = torch.ones(2, 2)
    with pytest.raises(ql.QuantizeError, match="at least 1 dimension"):
        ql.matmul(torch.ones(()), x)
    with pytest.raises(ql.QuantizeError, match="__matmul__"):
        ql.matmul(x, x.half())
    with pytest.raises(ql.QuantizeError, match="__matmul__"):
        ql.matmul(x.to(torch.int8), x.to(torch.int8))
