"""Host-side logic of the multi-GPU paths with two CPU ranks over gloo: how columns are dealt to
ranks, that an all-gather of column shards rebuilds Y (config 4), and that summing the row-parallel
partial products over ranks gives the unsharded result (config 5).  The arithmetic on each rank is
the CPU oracle's: the product has no CPU path, this file tests the decomposition only."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    for p in (os.path.join(ROOT, "tensorrt-incubator_b200"), os.path.join(ROOT, "oracle")):
        sys.path.insert(0, p)
    import oracle as orc
    from qlinear.mlp import shard_range
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(5)  # same stream on every rank
    M, K, N = 16, 64, 48
    xq = rng.integers(0, 0x78, size=(M, K), dtype=np.uint8)
    wq = rng.integers(0, 0x78, size=(N, K), dtype=np.uint8)
    sx, sw = np.float32(0.01), (rng.random(N).astype(np.float32) * 0.01 + 0.001)
    full = orc.to_f32(orc.gemm_fp8(xq, wq, sx, sw, orc.BF16), orc.BF16)

    # config 4: column-parallel, all-gather of the [M, N/world] blocks
    a, b = shard_range(N, world, rank)
    local = orc.to_f32(orc.gemm_fp8(xq, wq[a:b], sx, sw[a:b], orc.BF16), orc.BF16)
    gathered = [torch.zeros(M, N // world) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(local))
    y = torch.cat(gathered, dim=1).numpy()
    ok_gather = np.array_equal(y, full)

    # config 5: row-parallel (K split), all-reduce of f32 partial products
    ka, kb = shard_range(K, world, rank)
    part = orc.gemm_fp8(np.ascontiguousarray(xq[:, ka:kb]), np.ascontiguousarray(wq[:, ka:kb]), sx, sw, orc.F32)
    t = torch.from_numpy(part.copy())
    dist.all_reduce(t)
    exact = orc.gemm_fp8(xq, wq, sx, sw, orc.F32)
    ok_reduce = np.allclose(t.numpy(), exact, rtol=1e-5, atol=1e-6)
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write(f"{int(ok_gather)} {int(ok_reduce)}")
    dist.destroy_process_group()


def test_shard_range():
    from qlinear.mlp import shard_range
    assert [shard_range(28672, 8, r) for r in (0, 7)] == [(0, 3584), (25088, 28672)]
    with pytest.raises(ValueError):
        shard_range(10, 3, 0)


def test_two_rank_gather_and_reduce(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f"rank{r}.txt").read() == "1 1"
