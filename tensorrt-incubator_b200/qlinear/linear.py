"""Linear layer with quantized weights, mirroring Tripy's tp.Linear
(tripy/nvtripy/frontend/module/linear.py:60-151): same constructor arguments, same parameters
(weight [out, in], bias, weight_scale, input_scale) and the same forward semantics
    q_w = quantize(weight, weight_scale, quant_dtype, weight_quant_dim)
    out = x @ transpose(dequantize(q_w, weight_scale, dtype, weight_quant_dim)) (+ bias)
with the dequantize folded into the product: weights stay quantized in HBM and the scale is
applied to f32 partial sums.  Quantized weights are computed once and cached."""
from __future__ import annotations

import torch

from . import _lib
from . import dtypes as dt
from . import ops
from .tensor import Int4Tensor, current_stream, ql_view


class Linear:
    def __init__(self, in_features: int, out_features: int, bias: bool = True, dtype: dt.dtype = dt.float32,
                 quant_dtype: dt.dtype | None = None, weight_quant_dim: int | None = None, device="cuda"):
        self.in_features, self.out_features = in_features, out_features
        self.dtype = dtype
        self.quant_dtype = quant_dtype
        self.weight_quant_dim = weight_quant_dim
        self.weight = torch.zeros(out_features, in_features, dtype=dtype.torch, device=device)
        self.bias = torch.zeros(out_features, dtype=dtype.torch, device=device) if bias else None
        self.weight_scale = None
        self.input_scale = None
        self._qweight = None

    def __setattr__(self, name, value):
        # parameters may be assigned directly, as Tripy's tests do: keep them on the layer's device and drop the
        # cached quantized weight when what it was made from changes
        if name in ("weight", "bias", "weight_scale", "input_scale"):
            if isinstance(value, torch.Tensor) and "weight" in self.__dict__ and name != "input_scale":
                value = value.to(self.__dict__["weight"].device)
            self.__dict__["_qweight"] = None
        object.__setattr__(self, name, value)

    def load_state_dict(self, state: dict) -> None:
        for k, v in state.items():
            if k not in ("weight", "bias", "weight_scale", "input_scale"):
                raise KeyError(k)
            setattr(self, k, v if v is None else v.to(self.weight.device))
        self._qweight = None

    def quantized_weight(self):
        if self._qweight is None:
            self._qweight = ops.quantize(self.weight, self.weight_scale, self.quant_dtype, self.weight_quant_dim)
            self.__dict__["_qweight_fresh"] = True   # written by the kernel just launched: not yet "constant"
        return self._qweight

    def _weights_constant(self) -> bool:
        """False for the call that quantized the weights (its quantize kernel is the one preceding the linear kernel
        on the stream), True afterwards."""
        fresh = self.__dict__.get("_qweight_fresh", True)
        self.__dict__["_qweight_fresh"] = False
        return not fresh

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return self.forward(x)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features).contiguous()
        if self.quant_dtype is None:
            out = linear(x2, self.weight, bias=self.bias)
        else:
            if self.input_scale is not None and self.weight_quant_dim == 1:
                raise ops.QuantizeError(
                    "Unsupported quantization parameters for Linear module. weight_quant_dim cannot be 1 when "
                    f"input_scale is provided. input_scale={self.input_scale}, weight_quant_dim={self.weight_quant_dim}")
            out = self._quantized_forward(x2)
        return out.reshape(*lead, self.out_features)

    def _quantized_forward(self, x2: torch.Tensor) -> torch.Tensor:
        """The general branches add the bias in the kernel's epilogue, in f32, before the one rounding to `dtype`
        (the reference rounds the product to `dtype` and then adds the bias in `dtype`)."""
        qw = self.quantized_weight()
        ws = ops._as_scale(self.weight_scale, self.dtype).to(x2.device)
        if self.input_scale is not None and self.quant_dtype in (dt.float8, dt.int8):
            # both operands quantized: integer / fp8 product, scales (and bias) in the epilogue
            qx = ops.quantize(x2, self.input_scale, self.quant_dtype)
            sx = torch.as_tensor(self.input_scale, dtype=torch.float32, device=x2.device).reshape(())
            sw = ws.to(torch.float32).reshape(-1) if ws.dim() else ws.to(torch.float32).reshape(())
            return linear(qx, qw, sx, sw, self.bias, out_dtype=self.dtype)
        if self.input_scale is not None:
            # int4 with an input scale: the activation goes through quantize -> dequantize as the reference does
            qx = ops.quantize(x2, self.input_scale, self.quant_dtype)
            x2 = ops.dequantize(qx, self.input_scale, self.dtype)
        # the weight-only kernels (16-bit activations, weights dequantized in registers); their bias is added after
        fast, out = self.dtype is not dt.float32, None
        if fast and self.quant_dtype is dt.int8 and self.weight_quant_dim == 0 and self.in_features % 64 == 0:
            out = linear_w8a16(x2, qw, ws, weights_constant=self._weights_constant())
        elif fast and self.quant_dtype is dt.int4 and ws.dim() == 2 and ws.shape[0] == self.out_features \
                and self.in_features % 128 == 0 and (self.in_features // ws.shape[1]) % 128 == 0:
            out = linear_w4a16(x2, qw, ws, weights_constant=self._weights_constant())
        if out is not None:
            return out if self.bias is None else out + self.bias.unsqueeze(0)
        # remaining legal combinations: dequantize on the GPU, then the product in `dtype`
        w = ops.dequantize(qw, ws, self.dtype, self.weight_quant_dim)
        return linear(x2, w, bias=self.bias)


def _out(M, N, torch_dtype, device):
    return torch.empty((M, N), dtype=torch_dtype, device=device)


def linear_w8a16(x: torch.Tensor, wq: torch.Tensor, scale: torch.Tensor, out=None, weights_constant: bool = False) -> torch.Tensor:
    """Y = X . (Wq * scale[:, None])^T, Wq int8 [N, K], X f16/bf16 [M, K].  `weights_constant`: Wq and scale were
    written before the kernel preceding this call on the stream was launched (QL_WEIGHTS_CONSTANT)."""
    y = out if out is not None else _out(x.shape[0], wq.shape[0], x.dtype, x.device)
    tx, tw, ts, ty = ql_view(x), ql_view(wq), ql_view(scale), ql_view(y)
    _lib.check(_lib.lib().ql_linear_weight_only(tx, tw, ts, ty, _lib.WEIGHTS_CONSTANT if weights_constant else 0, current_stream(x.device)))
    return y


def linear_w4a16(x: torch.Tensor, wq: Int4Tensor, scale: torch.Tensor, out=None, weights_constant: bool = False) -> torch.Tensor:
    """Y = X . dequantize(Wq)^T, Wq int4 [N, K] packed, scale [N, K / block]; `weights_constant` as in linear_w8a16."""
    y = out if out is not None else _out(x.shape[0], wq.shape[0], x.dtype, x.device)
    tx, tw, ts, ty = ql_view(x), ql_view(wq), ql_view(scale), ql_view(y)
    _lib.check(_lib.lib().ql_linear_weight_only(tx, tw, ts, ty, _lib.WEIGHTS_CONSTANT if weights_constant else 0, current_stream(x.device)))
    return y


def gemm_fp8(xq, wq, sx, sw, out_dtype: dt.dtype = dt.bfloat16, out=None) -> torch.Tensor:
    """Y = (Xq . Wq^T) * sx * sw; Xq [M,K], Wq [N,K] e4m3; sx scalar or [M]; sw scalar or [N]."""
    y = out if out is not None else _out(xq.shape[0], wq.shape[0], out_dtype.torch, xq.device)
    tx, tw, tsx, tsw, ty = ql_view(xq), ql_view(wq), ql_view(sx), ql_view(sw), ql_view(y)
    _lib.check(_lib.lib().ql_gemm_fp8(tx, tw, tsx, tsw, ty, current_stream(xq.device)))
    return y


def gemm_i8(xq, wq, sx, sw, out_dtype: dt.dtype = dt.bfloat16, out=None) -> torch.Tensor:
    y = out if out is not None else _out(xq.shape[0], wq.shape[0], out_dtype.torch, xq.device)
    tx, tw, tsx, tsw, ty = ql_view(xq), ql_view(wq), ql_view(sx), ql_view(sw), ql_view(y)
    _lib.check(_lib.lib().ql_gemm_i8(tx, tw, tsx, tsw, ty, current_stream(xq.device)))
    return y


def gemm_16(x: torch.Tensor, w: torch.Tensor, sw=None, out=None) -> torch.Tensor:
    """Y = (X . W^T) * sw for f16 / bf16 operands ([M,K], [N,K])."""
    y = out if out is not None else _out(x.shape[0], w.shape[0], x.dtype, x.device)
    tx, tw, ty = ql_view(x), ql_view(w), ql_view(y)
    tsw = ql_view(sw) if sw is not None else None
    _lib.check(_lib.lib().ql_gemm_16(tx, tw, tsw, ty, current_stream(x.device)))
    return y


def linear(x: torch.Tensor, w: torch.Tensor, sx=None, sw=None, bias=None, out_dtype: dt.dtype | None = None, out=None) -> torch.Tensor:
    """Y = (X . W^T) * sx * sw + bias (ql_linear): X [M,K], W [N,K] of one type (f32, f16, bf16, e4m3, int8); any
    shape and alignment."""
    od = out_dtype.torch if out_dtype is not None else x.dtype
    y = out if out is not None else _out(x.shape[0], w.shape[0], od, x.device)
    v = lambda t: ql_view(t) if t is not None else None
    _lib.check(_lib.lib().ql_linear(ql_view(x), ql_view(w), v(sx), v(sw), v(bias), ql_view(y), current_stream(x.device)))
    return y


def matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """`a @ b` with Tripy's rules (tripy/nvtripy/frontend/ops/matmul.py:29-108): operands of one float type
    (float32, float16, bfloat16), at least 1-D; two vectors give a scalar, a vector on either side is a
    matrix-vector product, higher ranks are stacks of matrices whose leading dimensions broadcast."""
    da, db = dt.from_torch(a.dtype), dt.from_torch(b.dtype)
    if da not in dt.QUANTIZABLE_DTYPES or db is not da:
        raise ops.QuantizeError(f"Invalid inputs for function: '__matmul__'. Expected both operands to share one of "
                                f"{dt.QUANTIZABLE_DTYPES}, got {da} and {db}.")
    if a.dim() == 0 or b.dim() == 0:
        raise ops.QuantizeError(f"Input tensors must have at least 1 dimension. Note: Input tensors had {a.dim()} and {b.dim()} "
                                "dimension(s) respectively.")
    va, vb = a.dim() == 1, b.dim() == 1
    a2 = a.unsqueeze(0) if va else a
    b2 = b.unsqueeze(1) if vb else b
    if a2.shape[-1] != b2.shape[-2]:
        raise ops.QuantizeError(f"matmul: contracting dimensions differ ({a2.shape[-1]} and {b2.shape[-2]}).")
    rank = max(a2.dim(), b2.dim())
    a2 = a2.reshape((1,) * (rank - a2.dim()) + tuple(a2.shape))
    b2 = b2.reshape((1,) * (rank - b2.dim()) + tuple(b2.shape))
    lead = torch.broadcast_shapes(a2.shape[:-2], b2.shape[:-2])

    def lead_ok(t):   # all leading dimensions equal to the result's, or all 1
        return tuple(t.shape[:-2]) == tuple(lead) or all(d == 1 for d in t.shape[:-2])
    if not lead_ok(a2):
        a2 = a2.expand(*lead, *a2.shape[-2:])
    if not lead_ok(b2):
        b2 = b2.expand(*lead, *b2.shape[-2:])
    a2, b2 = a2.contiguous(), b2.contiguous()
    c = torch.empty(tuple(lead) + (a2.shape[-2], b2.shape[-1]), dtype=a.dtype, device=a.device)
    _lib.check(_lib.lib().ql_matmul(ql_view(a2), ql_view(b2), ql_view(c), current_stream(a.device)))
    if va:
        c = c.squeeze(-2)
    if vb:
        c = c.squeeze(-1)
    return c
