"""ctypes binding of lib/libqlinear_b200.so (declared in include/qlinear_b200.h).

The library is the only compute path.  If it has not been built, importing this module's
`lib()` raises: nothing here falls back to PyTorch or to the CPU.
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(HERE), "lib", "libqlinear_b200.so")

QL_MAX_RANK = 8

# ql_dtype
F32, F16, BF16, I8, I4, F8E4M3, F4E2M1 = 0, 1, 2, 3, 4, 5, 6
# ql_status
OK, ERR_INVALID_ARGUMENT, ERR_UNSUPPORTED, ERR_CUDA, ERR_NO_DEVICE, ERR_DEVICE_TIMEOUT = range(6)
# ql_fp8_mode
FP8_MODES = {"direct": 0, "via_f16": 1, "stablehlo": 2}


class QlError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


class QlTensor(ctypes.Structure):
    _fields_ = [
        ("data", ctypes.c_void_p),
        ("dtype", ctypes.c_int32),
        ("rank", ctypes.c_int32),
        ("shape", ctypes.c_int64 * QL_MAX_RANK),
    ]


class QlQdqAttrs(ctypes.Structure):
    _fields_ = [("has_axis", ctypes.c_int32), ("axis", ctypes.c_int32), ("fp8_mode", ctypes.c_int32)]


WEIGHTS_CONSTANT = 1  # flag of ql_linear_weight_only
PEER_NONE, PEER_STORE_ALL, PEER_ADD_ALL, PEER_ADD_OWNER = 0, 1, 2, 3  # ql_peer_mode
QL_MAX_PEERS = 8


class QlPeerBuffer(ctypes.Structure):
    _fields_ = [("replica", ctypes.c_void_p * QL_MAX_PEERS), ("all", ctypes.c_void_p), ("world", ctypes.c_int32),
                ("rank", ctypes.c_int32)]


_P = ctypes.POINTER(QlPeerBuffer)

# every symbol include/qlinear_b200.h declares, with its ctypes signature
_T = ctypes.POINTER(QlTensor)
_A = ctypes.POINTER(QlQdqAttrs)
_S = ctypes.c_void_p
SIGNATURES = {
    "ql_version": ([], ctypes.c_int),
    "ql_last_error": ([], ctypes.c_char_p),
    "ql_launch_count": ([], ctypes.c_uint64),
    "ql_device_info": ([ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32)], ctypes.c_int),
    "ql_quantize": ([_T, _T, _T, _A, _S], ctypes.c_int),
    "ql_dequantize": ([_T, _T, _T, _A, _S], ctypes.c_int),
    "ql_quantize_dequantize": ([_T, _T, _T, _T, _A, _S], ctypes.c_int),
    "ql_amax_scale": ([_T, _T, _A, ctypes.c_float, _S], ctypes.c_int),
    "ql_amax_scale_noalloc": ([_T, _T, _A, ctypes.c_float, _S], ctypes.c_int),
    "ql_dynamic_quantize": ([_T, _T, ctypes.c_int32, ctypes.c_int32, _T, _T, _S], ctypes.c_int),
    "ql_dequantize_nvfp4": ([_T, _T, _T, _T, _S], ctypes.c_int),
    "ql_gemm_nvfp4": ([_T, _T, _T, _T, _T, _T, _T, _S], ctypes.c_int),
    "ql_linear_w8a16": ([_T, _T, _T, _T, _S], ctypes.c_int),
    "ql_linear_w4a16": ([_T, _T, _T, _T, _S], ctypes.c_int),
    "ql_linear_weight_only": ([_T, _T, _T, _T, ctypes.c_uint32, _S], ctypes.c_int),
    "ql_gemm_fp8": ([_T, _T, _T, _T, _T, _S], ctypes.c_int),
    "ql_gemm_fp8_peer": ([_T, _T, _T, _T, _P, ctypes.c_int32, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, _S], ctypes.c_int),
    "ql_peer_barrier": ([_P, _S], ctypes.c_int),
    "ql_peer_reduce": ([_P, ctypes.c_int32, ctypes.c_int64, ctypes.c_int64, _S], ctypes.c_int),
    "ql_peer_broadcast": ([_P, ctypes.c_int64, ctypes.c_int64, _S], ctypes.c_int),
    "ql_gemm_i8": ([_T, _T, _T, _T, _T, _S], ctypes.c_int),
    "ql_gemm_16": ([_T, _T, _T, _T, _S], ctypes.c_int),
    "ql_linear": ([_T, _T, _T, _T, _T, _T, _S], ctypes.c_int),
    "ql_matmul": ([_T, _T, _T, _S], ctypes.c_int),
    "ql_set_peer_wait_limit": ([ctypes.c_int64], ctypes.c_int),
    "ql_rmsnorm_quant_fp8": ([_T, ctypes.c_float, _T, _T, _S], ctypes.c_int),
    "ql_swiglu_quant_fp8": ([_T, _T, _T, _S], ctypes.c_int),
    "ql_gemm_fp8_swiglu": ([_T, _T, _T, _T, _T, _T, _S], ctypes.c_int),
    "ql_quantize_rows_fp8": ([_T, _T, _T, _T, _S], ctypes.c_int),
    "ql_reload_tuning": ([], ctypes.c_int),
    "ql_gemm_status": ([ctypes.POINTER(ctypes.c_int32)], ctypes.c_int),
    "ql_nccl_version": ([ctypes.POINTER(ctypes.c_int32)], ctypes.c_int),
    "ql_nccl_unique_id": ([ctypes.c_void_p], ctypes.c_int),
    "ql_nccl_comm_init_rank": ([ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p, ctypes.c_int64,
                                ctypes.POINTER(ctypes.c_void_p)], ctypes.c_int),
    "ql_nccl_comm_split": ([ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.POINTER(ctypes.c_void_p)], ctypes.c_int),
    "ql_nccl_comm_rank": ([ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32)], ctypes.c_int),
    "ql_nccl_comm_destroy": ([ctypes.c_void_p], ctypes.c_int),
    "ql_nccl_all_reduce": ([ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint64, ctypes.c_int32, ctypes.c_int32, _S], ctypes.c_int),
    "ql_nccl_reduce_scatter": ([ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint64, ctypes.c_int32, ctypes.c_int32, _S], ctypes.c_int),
    "ql_nccl_all_gather": ([ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint64, _S], ctypes.c_int),
    "ql_nccl_all_to_all": ([ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint64, _S], ctypes.c_int),
    "ql_nccl_permute": ([ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_uint64, _S], ctypes.c_int),
}

_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python tensorrt-incubator_b200/build.py` "
                "(nvcc, sm_100a). There is no fallback path.")
        L = ctypes.CDLL(LIB_PATH)
        for name, (argtypes, restype) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.argtypes = argtypes
            fn.restype = restype
        _lib = L
    return _lib


def check(rc: int) -> None:
    if rc != OK:
        raise QlError(rc, lib().ql_last_error().decode("utf-8", "replace"))


def make_tensor(ptr: int, dtype: int, shape) -> QlTensor:
    t = QlTensor()
    t.data = ptr
    t.dtype = dtype
    shape = tuple(int(s) for s in shape)
    if len(shape) > QL_MAX_RANK:
        raise QlError(ERR_INVALID_ARGUMENT, f"rank {len(shape)} exceeds {QL_MAX_RANK}")
    t.rank = len(shape)
    for i, s in enumerate(shape):
        t.shape[i] = s
    return t


def make_attrs(axis=None, fp8_mode="direct") -> QlQdqAttrs:
    a = QlQdqAttrs()
    a.has_axis = 0 if axis is None else 1
    a.axis = 0 if axis is None else int(axis)
    a.fp8_mode = FP8_MODES[fp8_mode] if isinstance(fp8_mode, str) else int(fp8_mode)
    return a
