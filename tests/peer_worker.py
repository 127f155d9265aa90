"""One rank of the multi-GPU check of the fused GEMM + collective (run by tests/test_peer_gpu.py under
torchrun, one process per GPU).  Every rank draws the same operands from the same seed, so each can
compute the unsharded result by itself with the ordinary single-GPU GEMM and compare."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tensorrt-incubator_b200"))
import qlinear as ql  # noqa: E402
from qlinear import peer  # noqa: E402


def fp8(shape, seed, std, device):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=g) * std).to(torch.float8_e4m3fn).to(device)


def rel_err(got, want):
    got, want = got.float(), want.float()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-6))


def same_everywhere(t):
    """True when every rank holds the same bits."""
    mine = t.view(torch.int16).to(torch.int32).sum(dtype=torch.int64).reshape(1)
    lo, hi = mine.clone(), mine.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    return int(lo) == int(hi)


def check_nccl_entry_points(rank, world, dev):
    """The `ql_nccl_*` collectives of the C ABI between all ranks: the unique id travels over the process group, the
    results are compared with what each collective is defined to return."""
    from qlinear import nccl
    box = [nccl.unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    # a generous limit: the first point-to-point exchange of a communicator (all_to_all, permute) connects every pair of
    # ranks, which took longer than the default five seconds on eight GPUs
    comm = nccl.Communicator(rank, world, dev.index, box[0], timeout_ms=120000)
    assert (comm.rank, comm.num_ranks) == (rank, world)
    n = 4096
    mine = (torch.arange(n, device=dev) % 7 + rank).float()
    total = sum((torch.arange(n, device=dev) % 7 + r).float() for r in range(world))
    for dtype in (torch.float32, torch.bfloat16):
        out = torch.empty(n, dtype=dtype, device=dev)
        comm.all_reduce(mine.to(dtype), out)
        torch.cuda.synchronize()
        assert torch.equal(out.float(), total), f"rank {rank}: all_reduce {dtype}"
    out = torch.empty(n, device=dev)
    comm.all_reduce(mine, out, "max")
    torch.cuda.synchronize()
    assert torch.equal(out, (torch.arange(n, device=dev) % 7 + world - 1).float())
    part = torch.empty(n // world, device=dev)
    comm.reduce_scatter(mine, part)
    gathered = torch.empty(n * world, dtype=torch.int8, device=dev)
    comm.all_gather(torch.full((n,), rank, dtype=torch.int8, device=dev), gathered)
    sent = torch.arange(world, device=dev, dtype=torch.int32).repeat_interleave(16) + 100 * rank   # block p goes to rank p
    got = torch.empty_like(sent)
    comm.all_to_all(sent, got)
    ring = torch.empty(8, dtype=torch.int32, device=dev)
    comm.permute(torch.full((8,), rank, dtype=torch.int32, device=dev), ring, (rank + 1) % world, (rank - 1) % world)
    torch.cuda.synchronize()
    assert torch.equal(part, total[rank * (n // world):(rank + 1) * (n // world)])
    assert torch.equal(gathered.view(world, n)[:, 0].cpu(), torch.arange(world, dtype=torch.int8))
    assert torch.equal(got.view(world, 16)[:, 0].cpu(), torch.arange(world, dtype=torch.int32) * 100 + rank)
    assert int(ring[0]) == (rank - 1) % world
    half = comm.split(rank % 2, rank)      # even and odd ranks
    members = len(range(rank % 2, world, 2))
    assert half.num_ranks == members and half.rank == rank // 2
    s = torch.ones(4, device=dev)
    half.all_reduce(s, s)
    torch.cuda.synchronize()
    assert float(s[0]) == members
    half.destroy()
    comm.destroy()
    dist.barrier()
    if rank == 0:
        print("NCCL ABI OK")


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    check_nccl_entry_points(rank, world, dev)
    # Partial results are added rank by rank in bf16 (in the epilogue, in the switch, or by NCCL), each addition rounding
    # to 2^-9 of the running sum: the worst element may be off by (world - 1) such roundings on top of the benchmark's
    # 1e-2, the bound `bench.py` uses for its own check (0.015 on two ranks, 0.03 on eight; never below 0.02 here).
    tol = max(2e-2, 1e-2 + 0.0025 * world)
    if not peer.available():
        if rank == 0:
            print("PEER UNAVAILABLE")
        dist.destroy_process_group()
        return

    for (M, N, K) in [(256, 512, 512), (2048, 4096, 1024)]:     # one-CTA kernel; CTA-pair kernel
        xq, wq = fp8((M, K), 11, 1.0, dev), fp8((N, K), 12, 1.0, dev)
        sx = torch.rand(M, generator=torch.Generator().manual_seed(13)).add(0.5).to(dev)
        sw = torch.rand(N, generator=torch.Generator().manual_seed(14)).add(0.5).mul(1e-2).to(dev)
        full = ql.gemm_fp8(xq, wq, sx, sw)

        # column-parallel + store into every replica: bit-exact with the unsharded GEMM
        nl = N // world
        dest = peer.PeerTensor((M, N), torch.bfloat16)
        peer.gemm_fp8_peer(xq, wq[rank * nl:(rank + 1) * nl].contiguous(), sx, sw[rank * nl:(rank + 1) * nl].contiguous(),
                           dest, peer.STORE_ALL, col0=rank * nl)
        dest.barrier()
        torch.cuda.synchronize()
        assert torch.equal(dest.local, full), f"rank {rank}: STORE_ALL differs for {(M, N, K)}"

        # row-parallel (K split) + add into every replica: equals the unsharded GEMM up to bf16 rounding of the partial sums
        kl = K // world
        acc = peer.PeerTensor((M, N), torch.bfloat16)
        for _ in range(2):   # twice, to check the clear / barrier protocol as well
            acc.local.zero_()
            acc.barrier()
            peer.gemm_fp8_peer(xq[:, rank * kl:(rank + 1) * kl].contiguous(), wq[:, rank * kl:(rank + 1) * kl].contiguous(),
                               sx, sw, acc, peer.ADD_ALL)
            acc.barrier()
            torch.cuda.synchronize()
            e = rel_err(acc.local, full)
            assert e < tol, f"rank {rank}: ADD_ALL off by {e} for {(M, N, K)}"
        # reduce-scatter into the owners' rows, then the owners broadcast: the same sum again
        if M % (128 * world) == 0:
            rs = peer.PeerTensor((M, N), torch.bfloat16)
            rows = M // world
            peer.gemm_fp8_peer(xq[:, rank * kl:(rank + 1) * kl].contiguous(), wq[:, rank * kl:(rank + 1) * kl].contiguous(),
                               sx, sw, rs, peer.ADD_OWNER)
            rs.barrier()
            rs.broadcast_rows(rank * rows, rows)
            rs.barrier()
            torch.cuda.synchronize()
            e = rel_err(rs.local, full)
            assert e < tol, f"rank {rank}: ADD_OWNER + broadcast off by {e} for {(M, N, K)}"
            assert same_everywhere(rs.local), "replicas differ after ADD_OWNER + broadcast"
        # local partial results summed by the switch: one rounding, so at least as close as the bf16 adds above
        sw_buf = peer.PeerTensor((M, N), torch.bfloat16)
        if M % world == 0:
            rows = M // world
            ql.gemm_fp8(xq[:, rank * kl:(rank + 1) * kl].contiguous(), wq[:, rank * kl:(rank + 1) * kl].contiguous(), sx, sw, out=sw_buf.local)
            sw_buf.barrier()
            sw_buf.reduce_rows(rank * rows, rows)
            sw_buf.barrier()
            torch.cuda.synchronize()
            e = rel_err(sw_buf.local, full)
            assert e < tol, f"rank {rank}: in-switch reduce off by {e} for {(M, N, K)}"
            assert same_everywhere(sw_buf.local), "replicas differ after the in-switch reduce"
        # with two ranks a + b = b + a, so adding into every replica leaves them identical; with more ranks
        # the order of arrival differs per replica, which is why the MLP then uses owners
        if world == 2:
            assert same_everywhere(acc.local), "replicas differ after ADD_ALL"

    # the MLP block: fused all-reduce against the NCCL all-reduce on the same shards
    T, H, I = 1024, 1024, 2048
    il = I // world
    g = torch.Generator(device="cpu").manual_seed(100 + rank)
    def w(shape):
        return (torch.randn(shape, generator=g) * 0.02).to(torch.bfloat16).to(dev)
    wg, wu, wd = w((il, H)), w((il, H)), w((H, il))
    x = (torch.randn((T, H), generator=torch.Generator().manual_seed(5))).to(torch.bfloat16).to(dev)
    fused = ql.QuantizedMLP(wg, wu, wd, group=dist.group.WORLD, fused_all_reduce=True)
    plain = ql.QuantizedMLP(wg, wu, wd, group=dist.group.WORLD, fused_all_reduce=False)
    want = plain(x).clone()
    scattered = ql.QuantizedMLP(wg, wu, wd, group=dist.group.WORLD, fused_all_reduce="scatter")
    switched = ql.QuantizedMLP(wg, wu, wd, group=dist.group.WORLD, fused_all_reduce="switch")
    piped = ql.QuantizedMLP(wg, wu, wd, group=dist.group.WORLD, fused_all_reduce="pipeline")
    assert piped.protocol(T, dev) == "switch_pipelined"
    assert fused.protocol(T, dev) == ("add_all" if world == 2 else "add_owner")
    assert scattered.protocol(T, dev) == "add_owner" and switched.protocol(T, dev) == "switch_reduce"
    for name, mlp in (("auto", fused), ("add-owner", scattered), ("switch", switched), ("switch, pipelined over token slabs", piped)):
        for i in range(3):
            got = mlp(x)
            torch.cuda.synchronize()
            e = rel_err(got, want)
            assert e < tol, f"rank {rank}: fused MLP ({name}) call {i} off by {e}"
            assert same_everywhere(got), f"fused MLP ({name}) call {i}: ranks disagree"
    # Lifetime of the result: it is this rank's replica of one of a few internal buffers used in turn, promised intact
    # during the next call (so it can be read back while that call runs) and gone after the call after that.
    x2 = (torch.randn((T, H), generator=torch.Generator().manual_seed(6))).to(torch.bfloat16).to(dev)
    for name, mlp in (("auto", fused), ("add-owner", scattered), ("switch", switched), ("switch, pipelined over token slabs", piped), ("nccl", plain)):
        y1 = mlp(x)
        keep = y1.clone()
        y2 = mlp(x2)
        torch.cuda.synchronize()
        assert y2.data_ptr() != y1.data_ptr() and torch.equal(y1, keep), f"MLP ({name}): the previous result was disturbed by the next call"
        assert rel_err(y2, plain(x2)) < tol
    assert ql.lib().ql_gemm_status(None) == 0
    dist.barrier()
    if rank == 0:
        print("PEER OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
