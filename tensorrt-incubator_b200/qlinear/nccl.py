"""NCCL communicators and collectives through the C ABI (`ql_nccl_*`): the host-side mirror of the executor
runtime's NCCL module (executor/lib/Runtime/Backend/Lua/Modules/NCCL/NCCLModule.cpp:233-385 of the reference).
A compiled program names these collectives; the tensor-parallel MLP block of this package uses its own fused
kernels instead and does not come through here."""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from . import dtypes as dt
from .tensor import current_stream, require_cuda

UNIQUE_ID_BYTES = 128
OPS = {"sum": 0, "prod": 1, "min": 2, "max": 3, "avg": 4}


def version() -> int:
    v = ctypes.c_int32(0)
    _lib.check(_lib.lib().ql_nccl_version(ctypes.byref(v)))
    return v.value


def unique_id() -> bytes:
    """The 128 bytes rank 0 creates and hands to every rank of a new communicator."""
    buf = ctypes.create_string_buffer(UNIQUE_ID_BYTES)
    _lib.check(_lib.lib().ql_nccl_unique_id(buf))
    return buf.raw


def _bytes(t: torch.Tensor) -> int:
    return t.numel() * t.element_size()


class Communicator:
    """One rank's end of an NCCL communicator.  `timeout_ms` bounds every wait for the communicator after a call
    (5000 ms, the reference's value, when 0)."""

    def __init__(self, rank: int, num_ranks: int, device: int, uid: bytes, timeout_ms: int = 0, _handle=None):
        if _handle is not None:
            self._h = _handle
        else:
            if len(uid) != UNIQUE_ID_BYTES:
                raise _lib.QlError(_lib.ERR_INVALID_ARGUMENT, f"a unique id is {UNIQUE_ID_BYTES} bytes, got {len(uid)}")
            h = ctypes.c_void_p()
            _lib.check(_lib.lib().ql_nccl_comm_init_rank(rank, num_ranks, device, ctypes.c_char_p(uid), timeout_ms, ctypes.byref(h)))
            self._h = h
        r, n = ctypes.c_int32(0), ctypes.c_int32(0)
        _lib.check(_lib.lib().ql_nccl_comm_rank(self._h, ctypes.byref(r), ctypes.byref(n)))
        self.rank, self.num_ranks = r.value, n.value

    def split(self, color: int, key: int):
        h = ctypes.c_void_p()
        _lib.check(_lib.lib().ql_nccl_comm_split(self._h, color, key, ctypes.byref(h)))
        return Communicator(0, 0, 0, b"", _handle=h) if h.value else None

    def destroy(self) -> None:
        if self._h is not None:
            h, self._h = self._h, None
            _lib.check(_lib.lib().ql_nccl_comm_destroy(h))

    def _reduce_args(self, send, recv, op):
        require_cuda(send, "send")
        require_cuda(recv, "recv")
        if send.dtype != recv.dtype or not send.is_contiguous() or not recv.is_contiguous():
            raise _lib.QlError(_lib.ERR_INVALID_ARGUMENT, "send and recv must be contiguous tensors of one element type")
        return dt.from_torch(send.dtype).code, OPS[op]

    def all_reduce(self, send: torch.Tensor, recv: torch.Tensor, op: str = "sum") -> torch.Tensor:
        code, o = self._reduce_args(send, recv, op)
        if recv.numel() != send.numel():
            raise _lib.QlError(_lib.ERR_INVALID_ARGUMENT, "all_reduce: recv must have as many elements as send")
        _lib.check(_lib.lib().ql_nccl_all_reduce(self._h, send.data_ptr(), recv.data_ptr(), send.numel(), code, o, current_stream(send.device)))
        return recv

    def reduce_scatter(self, send: torch.Tensor, recv: torch.Tensor, op: str = "sum") -> torch.Tensor:
        code, o = self._reduce_args(send, recv, op)
        if recv.numel() * self.num_ranks != send.numel():
            raise _lib.QlError(_lib.ERR_INVALID_ARGUMENT, "reduce_scatter: send must hold num_ranks times recv")
        _lib.check(_lib.lib().ql_nccl_reduce_scatter(self._h, send.data_ptr(), recv.data_ptr(), recv.numel(), code, o, current_stream(send.device)))
        return recv

    def all_gather(self, send: torch.Tensor, recv: torch.Tensor) -> torch.Tensor:
        require_cuda(send, "send")
        require_cuda(recv, "recv")
        if _bytes(recv) != _bytes(send) * self.num_ranks or not send.is_contiguous() or not recv.is_contiguous():
            raise _lib.QlError(_lib.ERR_INVALID_ARGUMENT, "all_gather: recv must hold num_ranks times send, both contiguous")
        _lib.check(_lib.lib().ql_nccl_all_gather(self._h, send.data_ptr(), recv.data_ptr(), _bytes(send), current_stream(send.device)))
        return recv

    def all_to_all(self, send: torch.Tensor, recv: torch.Tensor) -> torch.Tensor:
        require_cuda(send, "send")
        require_cuda(recv, "recv")
        if _bytes(recv) != _bytes(send) or not send.is_contiguous() or not recv.is_contiguous():
            raise _lib.QlError(_lib.ERR_INVALID_ARGUMENT, "all_to_all: send and recv must be contiguous and of one size")
        _lib.check(_lib.lib().ql_nccl_all_to_all(self._h, send.data_ptr(), recv.data_ptr(), _bytes(send), current_stream(send.device)))
        return recv

    def permute(self, send: torch.Tensor, recv: torch.Tensor, send_to: int, recv_from: int) -> torch.Tensor:
        require_cuda(send, "send")
        require_cuda(recv, "recv")
        if _bytes(recv) != _bytes(send) or not send.is_contiguous() or not recv.is_contiguous():
            raise _lib.QlError(_lib.ERR_INVALID_ARGUMENT, "permute: send and recv must be contiguous and of one size")
        _lib.check(_lib.lib().ql_nccl_permute(self._h, send.data_ptr(), recv.data_ptr(), send_to, recv_from, _bytes(send), current_stream(send.device)))
        return recv
