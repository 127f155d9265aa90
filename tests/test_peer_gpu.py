"""Fused GEMM + collective over the GPUs of one box: column-parallel GEMM whose epilogue assembles Y on
every GPU, row-parallel GEMM whose epilogue sums into every GPU's output, and the tensor-parallel MLP on
top of them.  Needs at least two GPUs; the ranks are child processes (tests/peer_worker.py)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_fused_collectives_all_gpus_of_the_box():
    import torch
    n = min(torch.cuda.device_count(), 8)
    if n < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n), "--master-addr", "127.0.0.1",
           "--master-port", "29571", os.path.join(ROOT, "tests", "peer_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    out = r.stdout + r.stderr
    print(out[-12000:])   # kept in the test log: which ranks ran, what they reported and, on failure, the first traceback
    assert r.returncode == 0, out[-12000:]
    assert "NCCL ABI OK" in out, out[-3000:]
    if "PEER UNAVAILABLE" in out:
        pytest.skip("no NVSwitch replication on this box")
    assert "PEER OK" in out, out[-3000:]
