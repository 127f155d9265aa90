"""ctypes/numpy front end of the CPU oracle (oracle/ql_oracle.c).  TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the benchmark's CPU-baseline leg import this module; the
product package never does.  Arrays are numpy; 16-bit float types without a numpy dtype
(bfloat16) travel as ``uint16`` bit patterns together with an explicit type code.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_build", "libql_oracle.so")
REF_LIB_PATH = os.path.join(HERE, "_ref", "libref_datatypes.so")

# element type codes of ql_oracle.c
F32, F16, BF16, I8, I4, F8E4M3 = 0, 1, 2, 3, 4, 5
PER_TENSOR, PER_CHANNEL, BLOCK = 0, 1, 2
FP8_DIRECT, FP8_VIA_F16, FP8_STABLEHLO = 0, 1, 2

_NP_OF = {F32: np.float32, F16: np.float16, BF16: np.uint16, I8: np.int8, I4: np.uint8, F8E4M3: np.uint8}
MAXBOUND = {I8: 127.0, I4: 7.0, F8E4M3: 448.0}


def build(force: bool = False) -> None:
    """Compile the oracle (and the reference's number types when the reference is present)."""
    src = os.path.join(HERE, "ql_oracle.c")
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
        env = dict(os.environ)
        env.pop("CC", None)
        env.pop("CXX", None)
        subprocess.run(["make", "-C", HERE], check=True, env=env, stdout=subprocess.DEVNULL)


_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(LIB_PATH)
        i64, vp, ci, f = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        L.orc_quantize.argtypes = [vp, ci, vp, ci, vp, ci, ci, i64, i64, i64, ci, i64, ci]
        L.orc_dequantize.argtypes = [vp, ci, vp, ci, vp, ci, ci, i64, i64, i64, ci, i64]
        L.orc_amax.argtypes = [vp, ci, vp, ci, i64, i64, i64, ci, i64]
        L.orc_scale_from_amax.argtypes = [vp, i64, f, vp, ci]
        L.orc_linear_w8.argtypes = [vp, ci, vp, vp, ci, i64, i64, i64, vp, ci, ci]
        L.orc_linear_w4.argtypes = [vp, ci, vp, vp, ci, i64, i64, i64, i64, vp, ci, ci]
        L.orc_matmul.argtypes = [vp, vp, vp, ci, i64, i64, i64, i64, i64, i64, i64, i64, i64, i64, vp, ci]
        L.orc_gemm_fp8.argtypes = [vp, vp, vp, i64, vp, i64, i64, i64, i64, vp, ci, ci]
        L.orc_gemm_i8.argtypes = [vp, vp, vp, i64, vp, i64, i64, i64, i64, vp, ci]
        L.orc_rmsnorm_quant_fp8.argtypes = [vp, ci, i64, i64, f, vp, vp]
        L.orc_swiglu_quant_fp8.argtypes = [vp, ci, i64, i64, vp, vp]
        L.orc_swiglu_interleaved.argtypes = [vp, i64, i64, vp, ci, vp]
        L.orc_f32_to_f8e4m3.argtypes = [f]
        L.orc_f32_to_f8e4m3.restype = ctypes.c_uint8
        L.orc_f8e4m3_to_f32.argtypes = [ctypes.c_uint8]
        L.orc_f8e4m3_to_f32.restype = f
        L.orc_f32_to_f16.argtypes = [f]
        L.orc_f32_to_f16.restype = ctypes.c_uint16
        L.orc_f16_to_f32.argtypes = [ctypes.c_uint16]
        L.orc_f16_to_f32.restype = f
        L.orc_f32_to_bf16.argtypes = [f]
        L.orc_f32_to_bf16.restype = ctypes.c_uint16
        L.orc_silu_mul.argtypes = [f, f]
        L.orc_silu_mul.restype = f
        L.orc_num_threads.restype = ci
        L.orc_dynamic_quantize_nvfp4.argtypes = [vp, ci, i64, i64, f, vp, vp]
        L.orc_dequantize_nvfp4.argtypes = [vp, vp, f, i64, i64, vp, ci]
        L.orc_f32_to_f4e2m1.argtypes = [f]
        L.orc_f32_to_f4e2m1.restype = ctypes.c_uint8
        L.orc_f4e2m1_to_f32.argtypes = [ctypes.c_uint8]
        L.orc_f4e2m1_to_f32.restype = f
        _lib = L
    return _lib


def ref_lib():
    """The reference's own DataTypes.cpp behind C wrappers, or None when it was never built."""
    global _ref
    if _ref is None and os.path.exists(REF_LIB_PATH):
        R = ctypes.CDLL(REF_LIB_PATH)
        f = ctypes.c_float
        R.ref_f32_to_f8e4m3.argtypes = [f]
        R.ref_f32_to_f8e4m3.restype = ctypes.c_uint8
        R.ref_f8e4m3_to_f32.argtypes = [ctypes.c_uint8]
        R.ref_f8e4m3_to_f32.restype = f
        R.ref_f32_to_f16.argtypes = [f]
        R.ref_f32_to_f16.restype = ctypes.c_uint16
        R.ref_f16_to_f32.argtypes = [ctypes.c_uint16]
        R.ref_f16_to_f32.restype = f
        R.ref_f32_to_bf16.argtypes = [f]
        R.ref_f32_to_bf16.restype = ctypes.c_uint16
        R.ref_bf16_to_f32.argtypes = [ctypes.c_uint16]
        R.ref_bf16_to_f32.restype = f
        R.ref_int4_saturate.argtypes = [ctypes.c_int]
        R.ref_int4_saturate.restype = ctypes.c_int
        for name in ("ref_f32_to_f8e4m3_n", "ref_f32_to_f16_n", "ref_f32_to_bf16_n"):
            getattr(R, name).argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64]
        _ref = R
    return _ref


def _ptr(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(ctypes.c_void_p)


def as_code(a: np.ndarray, code: int | None = None) -> int:
    if code is not None:
        return code
    return {np.dtype(np.float32): F32, np.dtype(np.float16): F16, np.dtype(np.int8): I8}[a.dtype]


def to_f32(a: np.ndarray, code: int) -> np.ndarray:
    """Exact widening of f32 / f16 / bf16-bits arrays to float32."""
    if code == F32:
        return a.astype(np.float32)
    if code == F16:
        return a.view(np.float16).astype(np.float32)
    if code == BF16:
        return (a.view(np.uint16).astype(np.uint32) << 16).view(np.float32)
    raise ValueError(code)


def from_f32(a: np.ndarray, code: int) -> np.ndarray:
    """Round a float32 array to f16 (np.float16) / bf16 (uint16 bits), ties to even."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    if code == F32:
        return a
    if code == F16:
        return a.astype(np.float16)
    if code == BF16:
        u = a.view(np.uint32)
        nan = (u & 0x7FFFFFFF) > 0x7F800000
        r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
        r[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)
        return r
    raise ValueError(code)


def _geom(shape, mode, axis, scale_shape):
    """Map (shape, mode, axis) to the oracle's (outer, C, inner, block_dim, block)."""
    shape = tuple(int(s) for s in shape)
    n = int(np.prod(shape)) if shape else 1
    if mode == PER_TENSOR:
        return n, 1, 1, 0, 1
    if mode == PER_CHANNEL:
        outer = int(np.prod(shape[:axis])) if axis > 0 else 1
        inner = int(np.prod(shape[axis + 1:])) if axis + 1 < len(shape) else 1
        return outer, shape[axis], inner, 0, 1
    rows, cols = shape
    srows, scols = scale_shape
    if scols == cols:
        return rows, cols, 1, 0, rows // srows
    assert srows == rows
    return rows, cols, 1, 1, cols // scols


def quantize(x, x_code, scale, s_code, q_code, mode=PER_TENSOR, axis=None, fp8_mode=FP8_DIRECT):
    x = np.ascontiguousarray(x)
    scale = np.ascontiguousarray(scale)
    outer, C, inner, bd, blk = _geom(x.shape, mode, axis, scale.shape)
    n = outer * C * inner
    if q_code == I4:
        q = np.zeros((n + 1) // 2, dtype=np.uint8)
    else:
        q = np.zeros(x.shape, dtype=_NP_OF[q_code])
    rc = lib().orc_quantize(_ptr(x), x_code, _ptr(scale), s_code, _ptr(q), q_code, mode, outer, C, inner, bd, blk, fp8_mode)
    assert rc == 0
    return q


def dequantize(q, q_code, scale, s_code, y_code, shape, mode=PER_TENSOR, axis=None):
    q = np.ascontiguousarray(q)
    scale = np.ascontiguousarray(scale)
    outer, C, inner, bd, blk = _geom(shape, mode, axis, scale.shape)
    y = np.zeros(shape, dtype=_NP_OF[y_code])
    rc = lib().orc_dequantize(_ptr(q), q_code, _ptr(scale), s_code, _ptr(y), y_code, mode, outer, C, inner, bd, blk)
    assert rc == 0
    return y


def amax(x, x_code, mode=PER_TENSOR, axis=None, scale_shape=None):
    x = np.ascontiguousarray(x)
    outer, C, inner, bd, blk = _geom(x.shape, mode, axis, scale_shape)
    if mode == PER_TENSOR:
        out = np.zeros((), dtype=np.float32)
    elif mode == PER_CHANNEL:
        out = np.zeros(C, dtype=np.float32)
    else:
        out = np.zeros(scale_shape, dtype=np.float32)
    lib().orc_amax(_ptr(x), x_code, _ptr(out), mode, outer, C, inner, bd, blk)
    return out


def scale_from_amax(am, maxbound, s_code):
    am = np.ascontiguousarray(am, dtype=np.float32)
    out = np.zeros(am.shape, dtype=_NP_OF[s_code])
    lib().orc_scale_from_amax(_ptr(am), am.size, float(maxbound), _ptr(out), s_code)
    return out


def linear_w8(X, x_code, Wq, scale, s_code, y_code, acc64=True):
    M, K = X.shape
    N = Wq.shape[0]
    Y = np.zeros((M, N), dtype=_NP_OF[y_code])
    lib().orc_linear_w8(_ptr(np.ascontiguousarray(X)), x_code, _ptr(np.ascontiguousarray(Wq)),
                        _ptr(np.ascontiguousarray(scale)), s_code, M, N, K, _ptr(Y), y_code, int(acc64))
    return Y


def linear_w4(X, x_code, Wp, scale, s_code, y_code, block, acc64=True):
    M, K = X.shape
    N = scale.shape[0]
    Y = np.zeros((M, N), dtype=_NP_OF[y_code])
    lib().orc_linear_w4(_ptr(np.ascontiguousarray(X)), x_code, _ptr(np.ascontiguousarray(Wp)),
                        _ptr(np.ascontiguousarray(scale)), s_code, M, N, K, block, _ptr(Y), y_code, int(acc64))
    return Y


def matmul(a, b, code, acc64=False):
    """a @ b with numpy's rank rules, operands and result of the float type `code` (bit patterns for 16-bit types)."""
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    va, vb = a.ndim == 1, b.ndim == 1
    a2 = a[None, :] if va else a
    b2 = b[:, None] if vb else b
    lead = np.broadcast_shapes(a2.shape[:-2], b2.shape[:-2])
    a2 = np.ascontiguousarray(np.broadcast_to(a2, lead + a2.shape[-2:]))
    b2 = np.ascontiguousarray(np.broadcast_to(b2, lead + b2.shape[-2:]))
    M, K = a2.shape[-2:]
    N = b2.shape[-1]
    batch = int(np.prod(lead)) if lead else 1
    c = np.zeros(lead + (M, N), dtype=_NP_OF[code])
    lib().orc_matmul(_ptr(a2), _ptr(b2), None, code, batch, M, N, K, K, 1, N, 1, M * K, K * N, _ptr(c), int(acc64))
    if va:
        c = c.reshape(c.shape[:-2] + (N,))
    if vb:
        c = c.reshape(c.shape[:-1])
    return c


def linear_float(x, w, bias, code, acc64=False):
    """x @ transpose(w) (+ bias): x [M,K], w [N,K], bias [N] or None, all of the float type `code`."""
    x, w = np.ascontiguousarray(x), np.ascontiguousarray(w)
    M, K = x.shape
    N = w.shape[0]
    y = np.zeros((M, N), dtype=_NP_OF[code])
    bp = _ptr(np.ascontiguousarray(bias)) if bias is not None else None
    lib().orc_matmul(_ptr(x), _ptr(w), bp, code, 1, M, N, K, K, 1, 1, K, 0, 0, _ptr(y), int(acc64))
    return y


_Q_MODE_OF_RANK = {0: PER_TENSOR, 1: PER_CHANNEL, 2: BLOCK}


def linear_module(x, weight, bias, code, quant_code=None, weight_quant_dim=None, weight_scale=None, input_scale=None, acc64=False):
    """The forward of tp.Linear, op by op (tripy/nvtripy/frontend/module/linear.py:127-151): an optional
    quantize -> dequantize of the input (per tensor), quantize -> dequantize of the weight (mode from
    weight_quant_dim and the scale's rank), x @ transpose(weight), + bias.  Everything in the float type `code`."""
    if quant_code is not None:
        if input_scale is not None:
            if weight_quant_dim == 1:
                raise ValueError("Unsupported quantization parameters for Linear module.")
            s = from_f32(np.asarray(input_scale, dtype=np.float32).reshape(()), code)
            q = quantize(x, code, s, code, quant_code)
            x = dequantize(q, quant_code, s, code, code, x.shape)
        ws = np.asarray(weight_scale)
        mode = _Q_MODE_OF_RANK[ws.ndim]
        q = quantize(weight, code, ws, code, quant_code, mode, weight_quant_dim)
        weight = dequantize(q, quant_code, ws, code, code, weight.shape, mode, weight_quant_dim)
    return linear_float(x, weight, bias, code, acc64)


def gemm_fp8(Xq, Wq, sx, sw, y_code=BF16, acc64=True):
    M, K = Xq.shape
    N = Wq.shape[0]
    sx = np.ascontiguousarray(np.atleast_1d(sx), dtype=np.float32)
    sw = np.ascontiguousarray(np.atleast_1d(sw), dtype=np.float32)
    Y = np.zeros((M, N), dtype=_NP_OF[y_code])
    lib().orc_gemm_fp8(_ptr(np.ascontiguousarray(Xq)), _ptr(np.ascontiguousarray(Wq)), _ptr(sx), sx.size,
                       _ptr(sw), sw.size, M, N, K, _ptr(Y), y_code, int(acc64))
    return Y


def gemm_i8(Xq, Wq, sx, sw, y_code=BF16):
    M, K = Xq.shape
    N = Wq.shape[0]
    sx = np.ascontiguousarray(np.atleast_1d(sx), dtype=np.float32)
    sw = np.ascontiguousarray(np.atleast_1d(sw), dtype=np.float32)
    Y = np.zeros((M, N), dtype=_NP_OF[y_code])
    lib().orc_gemm_i8(_ptr(np.ascontiguousarray(Xq)), _ptr(np.ascontiguousarray(Wq)), _ptr(sx), sx.size,
                      _ptr(sw), sw.size, M, N, K, _ptr(Y), y_code)
    return Y


def rmsnorm_quant_fp8(X, x_code, eps=1e-5):
    M, H = X.shape
    Q = np.zeros((M, H), dtype=np.uint8)
    s = np.zeros(M, dtype=np.float32)
    lib().orc_rmsnorm_quant_fp8(_ptr(np.ascontiguousarray(X)), x_code, M, H, float(eps), _ptr(Q), _ptr(s))
    return Q, s


def swiglu_quant_fp8(GU, x_code):
    M, I2 = GU.shape
    Q = np.zeros((M, I2 // 2), dtype=np.uint8)
    s = np.zeros(M, dtype=np.float32)
    lib().orc_swiglu_quant_fp8(_ptr(np.ascontiguousarray(GU)), x_code, M, I2 // 2, _ptr(Q), _ptr(s))
    return Q, s


def interleave_gate_up(gate, up):
    """Rows of `gate` and `up` ([I, ...] each, I a multiple of 32) interleaved in groups of 32: the weight layout of
    the gate/up projection whose epilogue applies SwiGLU."""
    I = gate.shape[0]
    rest = gate.shape[1:]
    return np.ascontiguousarray(np.stack([gate.reshape((I // 32, 32) + rest), up.reshape((I // 32, 32) + rest)], axis=1).reshape((2 * I,) + rest))


def gemm_fp8_swiglu(Xq, Wq, sx, sw, y_code=BF16, acc64=True):
    """(act, row_amax) of the gate/up projection with interleaved weights `Wq` [2I, K] and SwiGLU applied to the
    unrounded f32 projection; act [M, I] of type y_code, row_amax f32 [M]."""
    gu = gemm_fp8(Xq, Wq, sx, sw, F32, acc64)
    M, N = gu.shape
    act = np.zeros((M, N // 2), dtype=_NP_OF[y_code])
    am = np.zeros(M, dtype=np.float32)
    lib().orc_swiglu_interleaved(_ptr(gu), M, N, _ptr(act), y_code, _ptr(am))
    return act, am


def quantize_rows_fp8(act, code, row_amax):
    """tensorrt.quantize per row with scale[t] = row_amax[t] / 448 (1 for an all-zero row): (q, scale)."""
    s = (np.asarray(row_amax, dtype=np.float32) / np.float32(448.0)).astype(np.float32)
    s[s == 0] = 1.0
    return quantize(act, code, s, F32, F8E4M3, PER_CHANNEL, 0), s


def dynamic_quantize_nvfp4(x, x_code, double_quant_scale=1.0):
    """tensorrt.dynamic_quantize over the last axis: (packed e2m1 bytes [..., K/2], e4m3 block scales [..., K/16])."""
    K = x.shape[-1]
    rows = x.size // K
    q = np.empty(x.shape[:-1] + (K // 2,), dtype=np.uint8)
    s = np.empty(x.shape[:-1] + (K // 16,), dtype=np.uint8)
    xc = np.ascontiguousarray(x)
    rc = lib().orc_dynamic_quantize_nvfp4(_ptr(xc), x_code, rows, K, float(double_quant_scale), _ptr(q), _ptr(s))
    assert rc == 0
    return q, s


def dequantize_nvfp4(q, scales, double_quant_scale, y_code):
    """e2m1 data * (e4m3 block scale * double_quant_scale) -> array of y_code, shape [..., K]."""
    K = q.shape[-1] * 2
    rows = q.size * 2 // K
    y = np.empty(q.shape[:-1] + (K,), dtype={F32: np.float32, F16: np.float16, BF16: np.uint16}[y_code])
    qc, sc = np.ascontiguousarray(q), np.ascontiguousarray(scales)
    rc = lib().orc_dequantize_nvfp4(_ptr(qc), _ptr(sc), float(double_quant_scale), rows, K, _ptr(y), y_code)
    assert rc == 0
    return y


def gemm_nvfp4(qa, sa, ga, qb, sb, gb):
    """dequantize_nvfp4(a) @ dequantize_nvfp4(b)^T in f64 (the reference's documented use of dynamic_quantize:
    dequantize twice, then matrix_multiply; TensorRTOps.td:3279-3358): qa [M, K/2] packed e2m1 bytes, sa [M, K/16] e4m3
    bits, ga the double-quantization scale; likewise b [N, ...].  Returns float64 [M, N]."""
    a = dequantize_nvfp4(qa, sa, ga, F32).astype(np.float64)
    b = dequantize_nvfp4(qb, sb, gb, F32).astype(np.float64)
    return a @ b.T


def f8_to_f32(bits: np.ndarray) -> np.ndarray:
    """e4m3 bit patterns -> float32 values."""
    L = lib()
    lut = np.array([L.orc_f8e4m3_to_f32(i) for i in range(256)], dtype=np.float32)
    return lut[bits]


def unpack_i4(p: np.ndarray, n: int) -> np.ndarray:
    """Packed int4 bytes (low nibble first) -> int8 values."""
    p = p.reshape(-1)
    lo = (p & 0xF).astype(np.int8)
    hi = (p >> 4).astype(np.int8)
    v = np.stack([lo, hi], axis=1).reshape(-1)[:n]
    return ((v ^ 8) - 8).astype(np.int8)
