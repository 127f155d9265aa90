"""A bounded device-side wait that runs out: the kernel returns, the failure is reported as
QL_ERR_DEVICE_TIMEOUT, and the context keeps working.

ql_peer_barrier is called on one GPU with a two-rank buffer whose second "replica" is just another local
array that nobody writes to, and with the wait limit lowered to about a millisecond: rank 1 never
arrives, so the wait gives up.  Nothing faults and nothing spins for long; no second process, no NVSwitch
replication address and no peer mapping is involved."""
import ctypes

import pytest
import torch

import qlinear as ql
from qlinear import _lib
from qlinear.tensor import current_stream

pytestmark = pytest.mark.gpu


def _status():
    code = ctypes.c_int32(-1)
    rc = _lib.lib().ql_gemm_status(ctypes.byref(code))
    return rc, code.value


def test_barrier_wait_runs_out_and_the_next_launch_works():
    L = _lib.lib()
    assert _status() == (_lib.OK, 0)
    mine = torch.zeros(3, dtype=torch.int32, device="cuda")     # flags of "rank 0": [rank 0 arrived, rank 1 arrived, calls]
    absent = torch.zeros(3, dtype=torch.int32, device="cuda")   # flags of a rank 1 that does not exist
    desc = _lib.QlPeerBuffer()
    desc.replica[0], desc.replica[1] = mine.data_ptr(), absent.data_ptr()
    desc.all, desc.world, desc.rank = 0, 2, 0
    L.ql_set_peer_wait_limit(2_000_000)   # about a millisecond of SM clock
    try:
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        _lib.check(L.ql_peer_barrier(desc, current_stream(mine.device)))
        t1.record()
        torch.cuda.synchronize()
        assert t0.elapsed_time(t1) < 200.0   # gave up after the lowered limit, not the ten-second default
    finally:
        L.ql_set_peer_wait_limit(0)
    rc, code = _status()
    assert rc == _lib.ERR_DEVICE_TIMEOUT and code == 7
    assert "gave up waiting" in L.ql_last_error().decode()
    # rank 0 did announce itself to both flag arrays before it waited
    assert mine.tolist() == [1, 0, 1] and absent.tolist()[0] == 1
    # the status is cleared by reading it, and the device still runs kernels of the library
    assert _status() == (_lib.OK, 0)
    x = torch.randn(64, 128, device="cuda")
    s = ql.amax_scale(x, ql.int8)
    assert torch.equal(ql.quantize(x, s, ql.int8), torch.clamp(torch.round(x / s), -128, 127).to(torch.int8))
    y = ql.gemm_16(x.to(torch.bfloat16), x.to(torch.bfloat16))
    torch.cuda.synchronize()
    assert _status() == (_lib.OK, 0) and tuple(y.shape) == (64, 64)
