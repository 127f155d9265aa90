"""Data types of the operator layer, named as Tripy names them
(tripy/nvtripy/common/datatype.py:95-105 of the reference): float32, float16, bfloat16 are the
quantizable types; int8, int4 and float8 (e4m3fn) the quantized ones."""
from __future__ import annotations

import torch

from . import _lib


class dtype:
    def __init__(self, name: str, code: int, torch_dtype, itemsize_bits: int):
        self.name = name
        self.code = code
        self.torch = torch_dtype
        self.bits = itemsize_bits

    def __repr__(self):
        return self.name


float32 = dtype("float32", _lib.F32, torch.float32, 32)
float16 = dtype("float16", _lib.F16, torch.float16, 16)
bfloat16 = dtype("bfloat16", _lib.BF16, torch.bfloat16, 16)
int8 = dtype("int8", _lib.I8, torch.int8, 8)
int4 = dtype("int4", _lib.I4, None, 4)
float8 = dtype("float8", _lib.F8E4M3, torch.float8_e4m3fn, 8)
float4 = dtype("float4", _lib.F4E2M1, None, 4)   # e2m1; only produced by dynamic_quantize

# plain types `cast` converts between (no kernel of this library involved)
int32 = dtype("int32", -1, torch.int32, 32)
int64 = dtype("int64", -1, torch.int64, 64)
bool = dtype("bool", -1, torch.bool, 8)  # noqa: A001  (Tripy's name)

QUANTIZABLE_DTYPES = (float32, float16, bfloat16)
QUANTIZED_DTYPES = (int8, int4, float8)
MAXBOUND = {int8: 127.0, int4: 7.0, float8: 448.0}

_BY_TORCH = {d.torch: d for d in (float32, float16, bfloat16, int8, float8, int32, int64, bool)}


def from_torch(t) -> dtype:
    try:
        return _BY_TORCH[t]
    except KeyError:
        raise TypeError(f"unsupported torch dtype {t}")
