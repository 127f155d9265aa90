"""Buffers that every GPU of a process group maps at once, and the fp8 GEMM whose epilogue writes into
them: the collective of a tensor-parallel layer done by the GEMM itself.

`PeerTensor` allocates one replica per rank through torch's symmetric memory (device memory and the
rendezvous are torch's; one process per GPU), which also asks the driver for an NVSwitch replication
address of the set.  `gemm_fp8_peer` hands the addresses to `ql_gemm_fp8_peer` (include/qlinear_b200.h),
whose epilogue stores every finished tile into all replicas, adds it into all replicas, or adds it into the
replica of the rank that owns its rows.  The kernels wait on no peer; ranks are ordered by `barrier()`
(`ql_peer_barrier`, a bounded flag exchange over peer memory).  The reference has no multi-GPU execution
of this path, so nothing here mirrors one of its interfaces."""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import _lib
from . import dtypes as dt
from .tensor import current_stream, ql_view

STORE_ALL, ADD_ALL, ADD_OWNER = _lib.PEER_STORE_ALL, _lib.PEER_ADD_ALL, _lib.PEER_ADD_OWNER


class PeerUnavailable(RuntimeError):
    """This box cannot replicate writes across the group's GPUs (no NVSwitch multicast, or one rank)."""


def available(group=None) -> bool:
    """True when the group spans several GPUs that the driver can join in one replication group."""
    if not (dist.is_available() and dist.is_initialized()) or not 2 <= dist.get_world_size(group) <= _lib.QL_MAX_PEERS:
        return False
    try:
        from torch._C._autograd import DeviceType
        from torch._C._distributed_c10d import _SymmetricMemory
        return bool(_SymmetricMemory.has_multicast_support(DeviceType.CUDA, torch.cuda.current_device()))
    except Exception:
        return False


class PeerTensor:
    """`shape`/`dtype` on every rank of `group`; `.local` is this rank's replica (an ordinary CUDA tensor,
    zero-filled).  Construction is collective and synchronises the ranks on the host."""

    def __init__(self, shape, dtype: torch.dtype, group=None):
        import torch.distributed._symmetric_memory as symm
        if not available(group):
            raise PeerUnavailable("no NVSwitch replication across this group's GPUs")
        self.group = group if group is not None else dist.group.WORLD
        dev = torch.device("cuda", torch.cuda.current_device())
        self.local = symm.empty(*shape, dtype=dtype, device=dev)
        self._handle = symm.rendezvous(self.local, self.group)
        self.world, self.rank = int(self._handle.world_size), int(self._handle.rank)
        self.desc = _lib.QlPeerBuffer()
        for r, ptr in enumerate(self._handle.buffer_ptrs):
            self.desc.replica[r] = int(ptr)
        self.desc.all = int(self._handle.multicast_ptr)
        self.desc.world, self.desc.rank = self.world, self.rank
        if not self.desc.all:
            raise PeerUnavailable("the driver gave no replication address for this buffer")
        self.local.zero_()
        # flags of ql_peer_barrier: one arrival counter per peer and this rank's call counter
        self._flags = None
        if dtype != torch.int32 or tuple(shape) != (self.world + 1,):
            self._flags = PeerTensor((self.world + 1,), torch.int32, self.group)
        torch.cuda.synchronize()
        dist.barrier(group=self.group)   # every replica is zeroed before any rank uses the set

    def barrier(self) -> None:
        """Work queued before this call on every rank's current stream is complete and visible before work
        queued after it starts on any rank."""
        flags = self._flags if self._flags is not None else self
        _lib.check(_lib.lib().ql_peer_barrier(flags.desc, current_stream(self.local.device)))

    def reduce_rows(self, row0: int, rows: int) -> None:
        """Replaces rows [row0, row0 + rows) of every replica by their sum over the replicas (formed in the switch,
        f32 accumulation).  Ranks call it on disjoint row ranges, between two barriers."""
        row_bytes = self.local.shape[1] * self.local.element_size()
        _lib.check(_lib.lib().ql_peer_reduce(self.desc, dt.from_torch(self.local.dtype).code, row0 * row_bytes, rows * row_bytes,
                                             current_stream(self.local.device)))

    def broadcast_rows(self, row0: int, rows: int) -> None:
        """Copies rows [row0, row0 + rows) of this rank's replica into every replica."""
        row_bytes = self.local.shape[1] * self.local.element_size()
        _lib.check(_lib.lib().ql_peer_broadcast(self.desc, row0 * row_bytes, rows * row_bytes, current_stream(self.local.device)))


def gemm_fp8_peer(xq, wq, sx, sw, dest: PeerTensor, mode: int, col0: int = 0) -> None:
    """(Xq . Wq^T) * sx * sw for this rank's operands, written to columns [col0, col0 + N) of `dest`: stored in
    every replica (`STORE_ALL`), added into every replica (`ADD_ALL`), or added into the replica of each
    row's owner (`ADD_OWNER`; rank r owns rows [r * M / world, (r + 1) * M / world))."""
    M, N = xq.shape[0], wq.shape[0]
    rows, ld = dest.local.shape
    if rows != M or col0 + N > ld:
        raise ValueError(f"a [{M}, {N}] result at column {col0} does not fit the [{rows}, {ld}] buffer")
    tx, tw, tsx, tsw = ql_view(xq), ql_view(wq), ql_view(sx), ql_view(sw)
    _lib.check(_lib.lib().ql_gemm_fp8_peer(tx, tw, tsx, tsw, dest.desc, dt.from_torch(dest.local.dtype).code, ld, col0, mode,
                                           current_stream(xq.device)))
