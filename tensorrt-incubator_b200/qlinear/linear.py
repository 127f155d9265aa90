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

    def load_state_dict(self, state: dict) -> None:
        for k, v in state.items():
            if k not in ("weight", "bias", "weight_scale", "input_scale"):
                raise KeyError(k)
            setattr(self, k, v if v is None else v.to(self.weight.device))
        self._qweight = None

    def quantized_weight(self):
        if self._qweight is None:
            self._qweight = ops.quantize(self.weight, self.weight_scale, self.quant_dtype, self.weight_quant_dim)
        return self._qweight

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return self.forward(x)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features).contiguous()
        if self.quant_dtype is None:
            out = gemm_16(x2, self.weight)
        else:
            if self.input_scale is not None and self.weight_quant_dim == 1:
                raise ops.QuantizeError(
                    "Unsupported quantization parameters for Linear module. weight_quant_dim cannot be 1 when "
                    f"input_scale is provided. input_scale={self.input_scale}, weight_quant_dim={self.weight_quant_dim}")
            out = self._quantized_forward(x2)
        if self.bias is not None:
            out = out + self.bias.unsqueeze(0)
        return out.reshape(*lead, self.out_features)

    def _quantized_forward(self, x2: torch.Tensor) -> torch.Tensor:
        qw = self.quantized_weight()
        ws = self.weight_scale
        if self.input_scale is not None:
            # both operands quantized: integer / fp8 tensor-core product, scales in the epilogue
            qx = ops.quantize(x2, self.input_scale, self.quant_dtype)
            sx = torch.as_tensor(self.input_scale, dtype=torch.float32, device=x2.device).reshape(())
            sw = ws.to(torch.float32).reshape(-1) if ws.dim() else ws.to(torch.float32).reshape(())
            if self.quant_dtype is dt.float8:
                return gemm_fp8(qx, qw, sx, sw, out_dtype=self.dtype)
            if self.quant_dtype is dt.int8:
                return gemm_i8(qx, qw, sx, sw, out_dtype=self.dtype)
        if self.quant_dtype is dt.int8 and self.weight_quant_dim == 0 and self.dtype is not dt.float32:
            return linear_w8a16(x2, qw, ws)
        if self.quant_dtype is dt.int4 and ws.dim() == 2 and ws.shape[0] == self.out_features \
                and self.dtype is not dt.float32 and (self.in_features // ws.shape[1]) % 128 == 0:
            return linear_w4a16(x2, qw, ws)
        # remaining legal combinations: dequantize on the GPU, then the 16-bit tensor-core product
        w = ops.dequantize(qw, ws, self.dtype, self.weight_quant_dim)
        return gemm_16(x2, w)


def _out(M, N, torch_dtype, device):
    return torch.empty((M, N), dtype=torch_dtype, device=device)


def linear_w8a16(x: torch.Tensor, wq: torch.Tensor, scale: torch.Tensor, out=None) -> torch.Tensor:
    """Y = X . (Wq * scale[:, None])^T, Wq int8 [N, K], X f16/bf16 [M, K]."""
    y = out if out is not None else _out(x.shape[0], wq.shape[0], x.dtype, x.device)
    tx, tw, ts, ty = ql_view(x), ql_view(wq), ql_view(scale), ql_view(y)
    _lib.check(_lib.lib().ql_linear_w8a16(tx, tw, ts, ty, current_stream(x.device)))
    return y


def linear_w4a16(x: torch.Tensor, wq: Int4Tensor, scale: torch.Tensor, out=None) -> torch.Tensor:
    """Y = X . dequantize(Wq)^T, Wq int4 [N, K] packed, scale [N, K / block]."""
    y = out if out is not None else _out(x.shape[0], wq.shape[0], x.dtype, x.device)
    tx, tw, ts, ty = ql_view(x), ql_view(wq), ql_view(scale), ql_view(y)
    _lib.check(_lib.lib().ql_linear_w4a16(tx, tw, ts, ty, current_stream(x.device)))
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
