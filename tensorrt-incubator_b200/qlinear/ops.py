"""Operator layer: quantize / dequantize with the signatures and argument contract of Tripy's
tp.quantize / tp.dequantize (tripy/nvtripy/frontend/ops/quantize.py:39-119,
dequantize.py:39-114, argument checks frontend/ops/utils.py:187-251), running the sm_100a
kernels through the C ABI.  Tensors are torch tensors in GPU memory; int4 results are
Int4Tensor.  Scales are constants, as in the reference: a Python number, a numpy array or a
torch tensor (host or device); they are rounded to the floating-point type of the data."""
from __future__ import annotations

import torch

from . import _lib
from . import dtypes as dt
from .tensor import Float4Tensor, Int4Tensor, current_stream, dtype_of, empty_quantized, ql_view, require_cuda


class QuantizeError(ValueError):
    """Argument-contract violation, worded as Tripy words it."""


def _as_scale(scale, float_dtype: dt.dtype) -> torch.Tensor:
    """The scale as a tensor of the data's floating-point type (still wherever it was)."""
    if isinstance(scale, torch.Tensor):
        if scale.dtype != float_dtype.torch:
            raise QuantizeError(
                f"Scale dtype does not match expected dtype. scale should have dtype={float_dtype}, got {scale.dtype}")
        return scale
    return torch.as_tensor(scale, dtype=torch.float64).to(float_dtype.torch)


def _float_dtype_or_none(t):
    try:
        return dtype_of(t)
    except TypeError:
        return None


def check_qdq_args(input, scale, dtype, dim, is_quantize: bool) -> None:
    """The checks of Tripy's check_qdq_args, same order, same wording."""
    valid_in = dt.QUANTIZABLE_DTYPES if is_quantize else dt.QUANTIZED_DTYPES
    valid_out = dt.QUANTIZED_DTYPES if is_quantize else dt.QUANTIZABLE_DTYPES
    op = "quantize op" if is_quantize else "dequantize op"
    try:
        in_dtype = dtype_of(input)
    except TypeError:
        in_dtype = None
    if in_dtype not in valid_in:
        raise QuantizeError(f"Input does not have a valid dtype in {op}. input.dtype must be one of {valid_in}, got {in_dtype}")
    if dtype not in valid_out:
        raise QuantizeError(f"Unsupported data type in {op}. Supported data types are: {valid_out}. Got dtype={dtype}")
    quantized = dtype if is_quantize else in_dtype
    rank_in = len(input.shape)
    rank_s = scale.dim()
    if dim is not None:
        if rank_s != 1:
            raise QuantizeError(f"If dim is given, scale must be a 1-D tensor in per-channel {op}. scale has rank={rank_s}.")
    elif rank_s == 2:
        if rank_in != 2:
            raise QuantizeError(f"Input must be a 2-D tensor in block-wise {op}. input has rank={rank_in}.")
        if quantized is not dt.int4:
            raise QuantizeError(f"Unsupported data type in block-wise {op}. Only `int4` is supported, got {quantized}")
    elif rank_s != 0:
        raise QuantizeError(f"Scale must be a scalar tensor in per-tensor {op}. scale has rank={rank_s}.")


def quantize(input: torch.Tensor, scale, dtype: dt.dtype, dim=None, *, fp8_mode: str = "direct", out=None):
    """output = clamp(round_half_even(input / scale)) as `dtype` (int8, int4 or float8).

    `dim` given: per-channel, scale is 1-D of input.shape[dim].  2-D scale: block-wise (int4).
    Otherwise scale is a scalar: per-tensor."""
    float_dtype = _float_dtype_or_none(input)
    if float_dtype not in dt.QUANTIZABLE_DTYPES:
        check_qdq_args(input, torch.zeros(()), dtype, dim, True)
    s = _as_scale(scale, float_dtype)
    check_qdq_args(input, s, dtype, dim, True)
    require_cuda(input, "input")
    s = s.to(input.device).contiguous()
    x = input.contiguous()
    q = out if out is not None else empty_quantized(x.shape, dtype, x.device)
    attrs = _lib.make_attrs(dim, fp8_mode)
    tx, ts, tq = ql_view(x), ql_view(s), ql_view(q)
    _lib.check(_lib.lib().ql_quantize(tx, ts, tq, attrs, current_stream(x.device)))
    return q


def quantize_to(input: torch.Tensor, scale: torch.Tensor, out, dim=None, *, fp8_mode: str = "direct"):
    """tensorrt.quantize into a preallocated output with a device-resident scale of any float type
    (the operator itself allows f32 scales for 16-bit data; only Tripy's layer ties the two)."""
    require_cuda(input, "input")
    require_cuda(scale, "scale")
    tx, ts, tq = ql_view(input), ql_view(scale), ql_view(out)
    _lib.check(_lib.lib().ql_quantize(tx, ts, tq, _lib.make_attrs(dim, fp8_mode), current_stream(input.device)))
    return out


def dequantize(input, scale, dtype: dt.dtype, dim=None, *, out=None) -> torch.Tensor:
    """output = input * scale as `dtype` (float32, float16 or bfloat16).  A `Float4Tensor` (NVFP4 data) takes block
    scales of its own rank along the last axis, as in the documented use of tensorrt.dynamic_quantize."""
    if isinstance(input, Float4Tensor):
        require_cuda(input, "input")
        s = scale.to(input.device).contiguous()
        y = out if out is not None else torch.empty(input.shape, dtype=dtype.torch, device=input.device)
        _lib.check(_lib.lib().ql_dequantize(ql_view(input), ql_view(s), ql_view(y), _lib.make_attrs(None), current_stream(input.device)))
        return y
    if dtype not in dt.QUANTIZABLE_DTYPES:
        check_qdq_args(input, torch.zeros(()), dtype, dim, False)
    s = _as_scale(scale, dtype)
    check_qdq_args(input, s, dtype, dim, False)
    require_cuda(input, "input")
    s = s.to(input.device).contiguous()
    q = input if isinstance(input, Int4Tensor) else input.contiguous()
    y = out if out is not None else torch.empty(tuple(q.shape), dtype=dtype.torch, device=q.device)
    attrs = _lib.make_attrs(dim)
    tq, ts, ty = ql_view(q), ql_view(s), ql_view(y)
    _lib.check(_lib.lib().ql_dequantize(tq, ts, ty, attrs, current_stream(q.device)))
    return y


def quantize_dequantize(input: torch.Tensor, scale, dtype: dt.dtype, dim=None, *, fp8_mode: str = "direct"):
    """(quantize(input), dequantize(quantize(input))) in one pass over the input."""
    float_dtype = _float_dtype_or_none(input)
    if float_dtype not in dt.QUANTIZABLE_DTYPES:
        check_qdq_args(input, torch.zeros(()), dtype, dim, True)
    s = _as_scale(scale, float_dtype)
    check_qdq_args(input, s, dtype, dim, True)
    require_cuda(input, "input")
    s = s.to(input.device).contiguous()
    x = input.contiguous()
    q = empty_quantized(x.shape, dtype, x.device)
    y = torch.empty_like(x)
    attrs = _lib.make_attrs(dim, fp8_mode)
    tx, ts, tq, ty = ql_view(x), ql_view(s), ql_view(q), ql_view(y)
    _lib.check(_lib.lib().ql_quantize_dequantize(tx, ts, tq, ty, attrs, current_stream(x.device)))
    return q, y


def amax_scale(input: torch.Tensor, dtype: dt.dtype, dim=None, block=None, *, scale_dtype: dt.dtype | None = None,
               out=None) -> torch.Tensor:
    """scale = max|input| / maxbound(dtype) per tensor, per channel along `dim`, or per block.

    `block` = (block_dim, block_size) for 2-D inputs.  The reference has no such operator (its
    scales are constants); the formula is the one its user guide gives for calibration."""
    require_cuda(input, "input")
    x = input.contiguous()
    sd = scale_dtype or dtype_of(x)
    if block is not None:
        bdim, bsize = block
        if x.dim() != 2:
            raise QuantizeError("Input must be a 2-D tensor in block-wise quantize op.")
        shape = list(x.shape)
        if shape[bdim] % bsize:
            raise QuantizeError(f"block size {bsize} does not divide dimension {bdim} of {tuple(x.shape)}")
        shape[bdim] //= bsize
        dim = None
    elif dim is not None:
        shape = [x.shape[dim]]
    else:
        shape = []
    s = out if out is not None else torch.empty(shape, dtype=sd.torch, device=x.device)
    attrs = _lib.make_attrs(dim)
    tx, ts = ql_view(x), ql_view(s)
    _lib.check(_lib.lib().ql_amax_scale(tx, ts, attrs, dt.MAXBOUND[dtype], current_stream(x.device)))
    return s


def cast(input, dtype: dt.dtype):
    """Tripy's `cast` (tripy/nvtripy/frontend/ops/cast.py:40-118): into int4 / float8 it is a per-tensor quantize
    with scale 1.0 (from float32), out of int4 / float8 a per-tensor dequantize with scale 1.0 to float32, followed
    by an ordinary conversion where the target is something else; int8 converts like any integer type.  The same
    combinations are refused: float8 -> int4 / int8, int8 -> float8, int4 -> float8 / int8 / int64."""
    src = dtype_of(input)
    if src is dtype:
        return input
    refused = {dt.float8: (dt.int4, dt.int8), dt.int8: (dt.float8,), dt.int4: (dt.float8, dt.int8, dt.int64)}
    if dtype in refused.get(src, ()):
        raise QuantizeError(f"Unsupported cast from {src} to {dtype}.")
    if src in (dt.int4, dt.float8) or (src is dt.int8 and dtype is dt.bool):
        input = dequantize(input, 1.0, dt.float32)
        if dtype is dt.float32:
            return input
    if dtype in (dt.int4, dt.float8):
        x = input if input.dtype == torch.float32 else input.to(torch.float32)
        return quantize(x, 1.0, dtype)
    return input.to(dtype.torch)


def _global_scale(value, device) -> torch.Tensor:
    t = value if isinstance(value, torch.Tensor) else torch.tensor(float(value), dtype=torch.float32)
    if t.dim() != 0:
        raise QuantizeError(f"double_quant_scale must be a scalar tensor, got rank={t.dim()}.")
    return t.to(device).contiguous()


def dynamic_quantize(input: torch.Tensor, double_quant_scale=1.0, axis: int = -1, block_size: int = 16):
    """tensorrt.dynamic_quantize (NVFP4; tensorrt/include/mlir-tensorrt-dialect/TensorRT/IR/TensorRTOps.td:3279-3358):
    returns (data, scales): `data` a Float4Tensor of the input's shape, `scales` e4m3 with one entry per block of 16
    along `axis`, scales = (max|block| / 6) / double_quant_scale, data = input / (scales * double_quant_scale)."""
    require_cuda(input, "input")
    x = input.contiguous()
    ax = axis if axis >= 0 else x.dim() + axis
    gs = _global_scale(double_quant_scale, x.device)
    shape = tuple(x.shape)
    last = shape[-1] if shape else 0
    data = Float4Tensor(torch.empty(max(x.numel() // 2, 0), dtype=torch.uint8, device=x.device), shape) if x.numel() % 2 == 0 else None
    if data is None:
        raise QuantizeError("shape(input)[axis] must be divisible by 16.")
    scales = torch.empty(shape[:-1] + (last // 16,), dtype=torch.float8_e4m3fn, device=x.device)
    _lib.check(_lib.lib().ql_dynamic_quantize(ql_view(x), ql_view(gs), ax, block_size, ql_view(data), ql_view(scales), current_stream(x.device)))
    return data, scales


def dequantize_nvfp4(data: Float4Tensor, scales: torch.Tensor, double_quant_scale=1.0, dtype: dt.dtype = dt.float32) -> torch.Tensor:
    """The inverse of dynamic_quantize: data * (scales * double_quant_scale) as `dtype` (the two tensorrt.dequantize
    steps of the operator's documented use, in one pass)."""
    require_cuda(data, "data")
    gs = _global_scale(double_quant_scale, data.device)
    y = torch.empty(data.shape, dtype=dtype.torch, device=data.device)
    sc = scales.contiguous()   # kept alive across the call: a view only borrows the pointer
    _lib.check(_lib.lib().ql_dequantize_nvfp4(ql_view(data), ql_view(sc), ql_view(gs), ql_view(y), current_stream(data.device)))
    return y


def gemm_nvfp4(a: Float4Tensor, a_scales: torch.Tensor, b: Float4Tensor, b_scales: torch.Tensor, a_global=None, b_global=None,
               out_dtype: dt.dtype = dt.bfloat16, out=None) -> torch.Tensor:
    """dequantize_nvfp4(a) @ dequantize_nvfp4(b)^T on the block-scaled tensor cores: a [M,K], b [N,K] and their e4m3
    block scales as dynamic_quantize returns them; `a_global` / `b_global` the double-quantization scales (None = 1)."""
    require_cuda(a, "a")
    require_cuda(b, "b")
    y = out if out is not None else torch.empty((a.shape[0], b.shape[0]), dtype=out_dtype.torch, device=a.device)
    # the scale tensors must outlive the call: a view only borrows the pointer
    ta = _global_scale(a_global, a.device) if a_global is not None else None
    tb = _global_scale(b_global, b.device) if b_global is not None else None
    sa, sb = a_scales.contiguous(), b_scales.contiguous()
    _lib.check(_lib.lib().ql_gemm_nvfp4(ql_view(a), ql_view(sa), ql_view(ta) if ta is not None else None, ql_view(b), ql_view(sb),
                                        ql_view(tb) if tb is not None else None, ql_view(y), current_stream(a.device)))
    return y
