"""Buffers that every GPU of a process group maps at once, and the fp8 GEMM whose epilogue writes into
all of them: the collective of a tensor-parallel layer done by the GEMM itself.

`PeerTensor` allocates one replica per rank through torch's symmetric memory (device memory and the
rendezvous are torch's; one process per GPU) and asks the driver for an NVSwitch replication address of
the set.  `gemm_fp8_peer` hands that address to `ql_gemm_fp8_peer` (include/qlinear_b200.h), whose
epilogue stores or adds every finished tile into all replicas with one posted write per 16 bytes.  The
kernel waits on no peer; ordering between ranks is the caller's, with `PeerTensor.barrier()` (a
one-element NCCL all-reduce on the current stream).  The reference has no multi-GPU execution of this
path, so nothing here mirrors one of its interfaces."""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import _lib
from . import dtypes as dt
from .tensor import current_stream, ql_view

STORE_ALL, ADD_ALL = _lib.PEER_STORE_ALL, _lib.PEER_ADD_ALL


class PeerUnavailable(RuntimeError):
    """This box cannot replicate writes across the group's GPUs (no NVSwitch multicast, or one rank)."""


def available(group=None) -> bool:
    """True when the group spans several GPUs that the driver can join in one replication group."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) < 2:
        return False
    try:
        from torch._C._distributed_c10d import _SymmetricMemory
        from torch._C._autograd import DeviceType
        return bool(_SymmetricMemory.has_multicast_support(DeviceType.CUDA, torch.cuda.current_device()))
    except Exception:
        return False


class PeerTensor:
    """`shape`/`dtype` on every rank of `group`; `.local` is this rank's replica (an ordinary CUDA tensor),
    `.switch_ptr` the address through which a write reaches all replicas."""

    def __init__(self, shape, dtype: torch.dtype, group=None):
        import torch.distributed._symmetric_memory as symm
        if not available(group):
            raise PeerUnavailable("no NVSwitch replication across this group's GPUs")
        self.group = group if group is not None else dist.group.WORLD
        self.local = symm.empty(*shape, dtype=dtype, device=torch.device("cuda", torch.cuda.current_device()))
        self._handle = symm.rendezvous(self.local, self.group)
        self.switch_ptr = int(self._handle.multicast_ptr)
        if not self.switch_ptr:
            raise PeerUnavailable("the driver gave no replication address for this buffer")
        self._token = torch.zeros(1, dtype=torch.float32, device=self.local.device)
        self.local.zero_()
        self.barrier()

    def address(self, row: int = 0, col: int = 0) -> int:
        """Replication address of element (row, col) of the 2-D buffer."""
        return self.switch_ptr + (row * self.local.shape[1] + col) * self.local.element_size()

    def barrier(self) -> None:
        """All ranks' work queued before this point on the current stream is done before any rank's work
        queued after it starts."""
        dist.all_reduce(self._token, group=self.group)


def gemm_fp8_peer(xq, wq, sx, sw, dest: PeerTensor, mode: int, col0: int = 0) -> None:
    """(Xq . Wq^T) * sx * sw, written to columns [col0, col0 + N) of every replica of `dest`:
    stored (`STORE_ALL`) or added to what is there (`ADD_ALL`)."""
    M, N = xq.shape[0], wq.shape[0]
    rows, ld = dest.local.shape
    if rows != M or col0 + N > ld:
        raise ValueError(f"a [{M}, {N}] result at column {col0} does not fit the [{rows}, {ld}] buffer")
    ty = _lib.make_tensor(dest.address(0, col0), dt.from_torch(dest.local.dtype).code, (M, N))
    tx, tw, tsx, tsw = ql_view(xq), ql_view(wq), ql_view(sx), ql_view(sw)
    _lib.check(_lib.lib().ql_gemm_fp8_peer(tx, tw, tsx, tsw, ty, ld, mode, current_stream(xq.device)))
