"""The NCCL entry points of the C ABI (`ql_nccl_*`, mirroring the executor runtime's NCCL module) on one GPU: a
communicator of one rank runs every collective (each then moves this rank's data to itself), and a communicator
whose second rank never joins must come back as a time-out status, not as a stuck call.  The multi-rank cases run in
tests/peer_worker.py on boxes with several GPUs."""
import time

import pytest
import torch

import qlinear as ql
from qlinear import nccl

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def comm():
    c = nccl.Communicator(0, 1, 0, nccl.unique_id())
    yield c
    c.destroy()


def test_version_and_rank(comm):
    assert nccl.version() >= 21800   # ncclCommSplit needs 2.18
    assert (comm.rank, comm.num_ranks) == (0, 1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16, torch.int8])
def test_collectives_of_one_rank_return_the_input(comm, dtype):
    g = torch.Generator(device="cpu").manual_seed(5)
    x = (torch.randn(3000, generator=g) * 20).to(dtype).cuda()
    for op in ("sum", "max", "min", "prod", "avg"):
        if dtype == torch.int8 and op == "avg":
            continue
        y = torch.zeros_like(x)
        comm.all_reduce(x, y, op)
        torch.cuda.synchronize()
        assert torch.equal(x, y), op
    y = torch.zeros_like(x)
    comm.reduce_scatter(x, y)
    z = torch.zeros_like(x)
    comm.all_gather(x, z)
    w = torch.zeros_like(x)
    comm.all_to_all(x, w)
    p = torch.zeros_like(x)
    comm.permute(x, p, 0, 0)
    torch.cuda.synchronize()
    assert torch.equal(x, y) and torch.equal(x, z) and torch.equal(x, w) and torch.equal(x, p)
    q = torch.full_like(x, 7)
    comm.permute(x, q, -1, -1)   # neither sends nor receives: the receive buffer is zeroed
    torch.cuda.synchronize()
    assert int(q.float().abs().sum()) == 0


def test_in_place_and_split(comm):
    x = torch.arange(1024, dtype=torch.float32, device="cuda")
    comm.all_reduce(x, x)
    torch.cuda.synchronize()
    assert float(x[1023]) == 1023.0
    child = comm.split(3, 0)
    assert child is not None and (child.rank, child.num_ranks) == (0, 1)
    y = torch.zeros_like(x)
    child.all_reduce(x, y, "max")
    torch.cuda.synchronize()
    assert torch.equal(x, y)
    child.destroy()
    assert comm.split(-1, 0) is None   # no colour: this rank is in no new communicator


def test_argument_rules(comm):
    x = torch.zeros(16, device="cuda")
    with pytest.raises(ql.QlError, match="as many elements"):
        comm.all_reduce(x, torch.zeros(8, device="cuda"))
    with pytest.raises(ql.QlError, match="unsupported element type"):
        q = torch.zeros(16, dtype=torch.float8_e4m3fn, device="cuda")
        comm.all_reduce(q, q.clone())
    with pytest.raises(KeyError):
        comm.all_reduce(x, x.clone(), "xor")
    with pytest.raises(ql.QlError, match="128 bytes"):
        nccl.Communicator(0, 1, 0, b"short")


def test_a_rank_that_never_joins_is_a_timeout_status():
    """Two ranks announced, one arrives: the non-blocking communicator stays in progress, the bounded poll gives up
    after its limit and the communicator is aborted.  Nothing runs on the GPU."""
    t0 = time.time()
    with pytest.raises(ql.QlError, match="timed out") as e:
        nccl.Communicator(0, 2, 0, nccl.unique_id(), timeout_ms=400)
    assert e.value.status == ql._lib.ERR_DEVICE_TIMEOUT
    assert time.time() - t0 < 60
    # the library and NCCL stay usable
    c = nccl.Communicator(0, 1, 0, nccl.unique_id())
    x = torch.ones(8, device="cuda")
    c.all_reduce(x, x)
    torch.cuda.synchronize()
    c.destroy()
