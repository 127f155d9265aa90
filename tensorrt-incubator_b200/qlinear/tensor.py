"""Tensor plumbing between torch (device memory, streams) and the C ABI."""
from __future__ import annotations

import math

import torch

from . import _lib
from . import dtypes as dt


class Int4Tensor:
    """Signed 4-bit values, two per byte with the first element in the low nibble (the layout the
    reference gives TensorRT: tensorrt/lib/Target/TensorRTEncodingOpInterface/NetworkEncoder.cpp:552-570).
    `packed` is a flat uint8 tensor of ceil(numel / 2) bytes; `shape` is the logical shape."""

    dtype = dt.int4

    def __init__(self, packed: torch.Tensor, shape):
        self.shape = tuple(int(s) for s in shape)
        n = math.prod(self.shape)
        assert packed.dtype == torch.uint8 and packed.numel() == (n + 1) // 2
        self.packed = packed.contiguous()

    @property
    def device(self):
        return self.packed.device

    def numel(self) -> int:
        return math.prod(self.shape)

    def unpack(self) -> torch.Tensor:
        """int8 tensor of the logical shape (a host-side convenience for tests)."""
        p = self.packed.to(torch.int16)
        lo = p & 0xF
        hi = (p >> 4) & 0xF
        v = torch.stack([lo, hi], dim=1).reshape(-1)[: self.numel()]
        return (((v ^ 8) - 8).to(torch.int8)).reshape(self.shape)

    @staticmethod
    def pack(values: torch.Tensor) -> "Int4Tensor":
        v = values.reshape(-1).to(torch.int16) & 0xF
        if v.numel() % 2:
            v = torch.cat([v, v.new_zeros(1)])
        packed = (v[0::2] | (v[1::2] << 4)).to(torch.uint8)
        return Int4Tensor(packed, values.shape)


class Float4Tensor:
    """e2m1 values, two per byte with the first element in the low nibble; `packed` is a flat uint8 tensor of
    numel / 2 bytes, `shape` the logical shape (last dimension a multiple of 16: NVFP4 blocks)."""

    dtype = dt.float4
    _VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)

    def __init__(self, packed: torch.Tensor, shape):
        self.shape = tuple(int(s) for s in shape)
        assert packed.dtype == torch.uint8 and packed.numel() * 2 == math.prod(self.shape)
        self.packed = packed.contiguous()

    @property
    def device(self):
        return self.packed.device

    def numel(self) -> int:
        return math.prod(self.shape)

    def unpack(self) -> torch.Tensor:
        """float32 tensor of the logical shape (a host-side convenience for tests)."""
        p = self.packed.to(torch.int64)
        codes = torch.stack([p & 0xF, (p >> 4) & 0xF], dim=1).reshape(-1)
        lut = torch.tensor(self._VALUES + tuple(-v for v in self._VALUES), dtype=torch.float32, device=codes.device)
        return lut[codes].reshape(self.shape)


def dtype_of(t) -> dt.dtype:
    if isinstance(t, Float4Tensor):
        return dt.float4
    if isinstance(t, Int4Tensor):
        return dt.int4
    return dt.from_torch(t.dtype)


def ql_view(t) -> _lib.QlTensor:
    """QlTensor over a CUDA torch tensor or Int4Tensor (no copy; the caller keeps `t` alive)."""
    if isinstance(t, Int4Tensor):
        return _lib.make_tensor(t.packed.data_ptr(), _lib.I4, t.shape)
    if isinstance(t, Float4Tensor):
        return _lib.make_tensor(t.packed.data_ptr(), _lib.F4E2M1, t.shape)
    if not t.is_contiguous():
        raise _lib.QlError(_lib.ERR_INVALID_ARGUMENT, "tensors must be contiguous (dense row-major)")
    return _lib.make_tensor(t.data_ptr(), dt.from_torch(t.dtype).code, t.shape)


def require_cuda(t, what: str) -> None:
    dev = t.device
    if dev.type != "cuda":
        raise _lib.QlError(_lib.ERR_NO_DEVICE, f"{what} must live in GPU memory (got {dev}); there is no CPU path")


def current_stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def empty_quantized(shape, qdtype: dt.dtype, device):
    if qdtype is dt.int4:
        n = math.prod(shape)
        return Int4Tensor(torch.empty((n + 1) // 2, dtype=torch.uint8, device=device), shape)
    return torch.empty(tuple(shape), dtype=qdtype.torch, device=device)
