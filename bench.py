#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1|c2|c3|c4|c5|nvfp4] [--impl reference]

One JSON line on stdout (rank 0).  A step is one pass of the workload over one batch of seeded
synthetic input already resident in HBM; `value` is device-timed throughput over exactly K steps,
`e2e` the same metric with the step's inputs copied from pinned host memory and its results read
back inside the timed region.  Default workload: benchmark config 5, the fp8 Llama-style MLP block
(4096 tokens, 8192 -> 28672 -> 8192), unsharded on one GPU and tensor-parallel over N GPUs (strong
scaling: the same block, split).  At N = 1 the line also carries the fused int8 quantize/dequantize
round trip of config 1 and the fp8 GEMM of config 4 as extra entries of `parts`, so that one run
records all three kinds of kernel; the other configs are selectable with --workload and are
otherwise covered by the parity tests.  Before anything is timed the step's result is checked
(`parity_check`): against the same block computed stage by stage through the plain entry points,
against the NCCL all-reduce variant on the same shards when N > 1, and for bit-identity across ranks;
a mismatch ends the run with a non-zero exit code.

`--impl reference` times the CPU restatement of the reference's host path (oracle/) with all host
threads on a bounded sample of the same workload.  The product path never touches oracle/.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "tensorrt-incubator_b200"))

L2_BYTES = 126 * 1024 * 1024

# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of each workload's dominant
# kernel, from the ncu captures summarised under profiles/ (None until a capture exists).
# dram__bytes_read.sum + dram__bytes_write.sum per launch of each part, from the ncu captures summarised under
# profiles/ (one B200, 1 GPU workloads; parts made of two kernels give the sum of both)
TRAFFIC = {
    "config1_int8_qdq_round_trip:fused_qdq": 99_742_976,      # output partly still dirty in L2 when the kernel ends
    "config2_w8a16_linear:M=1": 45_127_936, "config2_w8a16_linear:M=16": 45_264_640, "config2_w8a16_linear:M=128": 46_199_040,
    "config2_w8a16_linear:M=2048": 198_069_248,               # includes the 16-bit scratch copy of the weights, written and read back
    "config3_w4a16_linear:M=1": 8_668_416, "config3_w4a16_linear:M=8": 8_726_016, "config3_w4a16_linear:M=32": 8_924_160,
    "config4_fp8_w8a8_gemm:fp8_gemm": 1_593_066_736,
    "config5_fp8_mlp_block:rmsnorm_quant": 72_518_400, "config5_fp8_mlp_block:gate_up_gemm": 1_712_782_648,
    "config5_fp8_mlp_block:gate_up_gemm_swiglu": 1_246_894_040,   # weights streamed once per band of 2048 tokens (two bands)
    "config5_fp8_mlp_block:quantize_rows": 314_609_664,           # part of the output still dirty in L2 when the kernel ends
    "config5_fp8_mlp_block:swiglu_quant": 559_550_512, "config5_fp8_mlp_block:down_gemm": 1_051_541_624,
}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ----------------------------------------------------------------------------------------------
# clocks sampled during the timed region
# ----------------------------------------------------------------------------------------------
class ClockSampler:
    """SM clock and throttle reasons of one GPU, polled through NVML every few milliseconds from a
    thread while the timed region runs (reading settings only; nothing is changed)."""

    def __init__(self, index: int, period_s: float = 0.001):
        self.index, self.period = index, period_s
        self.mhz, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self.thread = None
        self.error = None

    def _run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            uuid = None
            try:
                import torch
                uuid = "GPU-" + str(torch.cuda.get_device_properties(self.index).uuid)
            except Exception:
                pass
            h = None
            if uuid:
                try:
                    h = nv.nvmlDeviceGetHandleByUUID(uuid.encode() if isinstance(uuid, str) else uuid)
                except Exception:
                    h = None
            if h is None:
                h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            names = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown, "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
                     "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown, "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap}
            while not self._stop.is_set():
                self.mhz.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                for n, bit in names.items():
                    if mask & bit:
                        self.reasons.add(n)
                time.sleep(self.period)
        except Exception as e:  # NVML missing: report it, never fail the bench
            self.error = repr(e)

    def start(self):
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def wait_ready(self, timeout_s: float = 5.0):
        t0 = time.time()
        while not self.mhz and self.error is None and time.time() - t0 < timeout_s:
            time.sleep(0.002)

    def stop(self):
        self._stop.set()
        if self.thread is not None:
            self.thread.join(timeout=2)
        m = sorted(self.mhz)
        out = {"sm_mhz": m[len(m) // 2] if m else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(m)}
        if self.error:
            out["error"] = self.error
        return out


# ----------------------------------------------------------------------------------------------
# workloads
# ----------------------------------------------------------------------------------------------
class Workload:
    """A workload owns its device buffers and knows its algorithmic work.

    parts(): list of (name, fn, flops, bytes, bound) -- the kernels of one step, each timed
    separately so that the dominant one can be reported against its roofline."""

    name = metric = unit = dtype = ""
    use_graphs = True    # replay captured CUDA graphs: device time without host launch gaps
    scaling = "weak"
    parallelism = "replicas only"


class W8A16Linear(Workload):
    """Config 2: W f16 [11008,4096] ~ N(0,0.02) quantized per output channel to int8 once (weights are
    constants of the compiled program); X bf16 [M,4096] ~ N(0,1); Y = X . dequant(W)^T, bf16."""

    name = "config2_w8a16_linear"
    metric = "quantized GEMM TFLOP/s (config 2: int8 per-channel weights, W8A16 linear, M in {1,16,128,2048})"
    unit = "TFLOP/s"
    dtype = "bf16 x int8 -> f32 accumulate -> bf16"
    N, K = 11008, 4096
    MS = (1, 16, 128, 2048)
    REPLICAS = 6  # 6 x 45 MB of weights cycled per launch: every launch finds its weights cold in L2

    def __init__(self, torch, ql, device, dist=None, seed=1002):
        self.torch, self.ql, self.device = torch, ql, device
        g = torch.Generator(device="cpu").manual_seed(seed)
        w = (torch.randn((self.N, self.K), generator=g, dtype=torch.float32) * 0.02).to(torch.float16).to(device)
        self.scale = ql.amax_scale(w, ql.int8, dim=0)
        q = ql.quantize(w, self.scale, ql.int8, 0)
        self.wq = [q] + [q.clone() for _ in range(self.REPLICAS - 1)]
        del w
        self.x_host = {m: torch.randn((m, self.K), generator=g, dtype=torch.float32).to(torch.bfloat16).pin_memory() for m in self.MS}
        self.x = {m: self.x_host[m].to(device) for m in self.MS}
        self.y = {m: torch.empty((m, self.N), dtype=torch.bfloat16, device=device) for m in self.MS}
        self.y_host = {m: torch.empty((m, self.N), dtype=torch.bfloat16).pin_memory() for m in self.MS}
        self.turn = 0

    def flops(self, m):
        return 2 * m * self.N * self.K

    def bytes(self, m):
        return self.N * self.K + self.N * 2 + m * self.K * 2 + m * self.N * 2

    def run_part(self, m):
        w = self.wq[self.turn % self.REPLICAS]
        self.turn += 1
        self.ql.linear_w8a16(self.x[m], w, self.scale, out=self.y[m], weights_constant=True)   # quantized once, in __init__

    def parts(self):
        return [(f"M={m}", (lambda m=m: self.run_part(m)), self.flops(m), self.bytes(m), "tensor" if m >= 512 else "hbm") for m in self.MS]

    def e2e_units(self, step):
        # one unit per batch size: each has its own device and host buffers
        return [(("x", m), ("y", m), (lambda m=m: self.x[m].copy_(self.x_host[m], non_blocking=True)), (lambda m=m: self.run_part(m)),
                 (lambda m=m: self.y_host[m].copy_(self.y[m], non_blocking=True))) for m in self.MS]

    def e2e_bytes(self):
        return sum(m * self.K * 2 for m in self.MS), sum(m * self.N * 2 for m in self.MS)

    def config(self):
        return {"workload": self.name, "N": self.N, "K": self.K, "M": list(self.MS), "weights": "int8 per-channel (axis 0), f16 scales",
                "l2": f"{self.REPLICAS} weight replicas ({self.REPLICAS * self.N * self.K >> 20} MiB > 126 MiB L2) cycled per launch",
                "seed": 1002}


class W4A16Linear(Workload):
    """Config 3: W f16 [4096,4096] ~ N(0,0.02) -> int4 in blocks of 128 along K (f16 scales, low nibble
    first); X f16 [M,4096]; Y = X . dequant(W)^T, f16; M in {1, 8, 32}."""

    name = "config3_w4a16_linear"
    metric = "quantized GEMM TFLOP/s (config 3: block-128 int4 weights, W4A16 linear, M in {1,8,32})"
    unit = "TFLOP/s"
    dtype = "f16 x int4 -> f32 accumulate -> f16"
    N, K, B = 4096, 4096, 128
    MS = (1, 8, 32)
    REPLICAS = 24  # 24 x 8.25 MiB of weights + scales cycled per launch (198 MiB > L2)

    def __init__(self, torch, ql, device, dist=None, seed=1003):
        self.torch, self.ql, self.device = torch, ql, device
        g = torch.Generator(device="cpu").manual_seed(seed)
        w = (torch.randn((self.N, self.K), generator=g, dtype=torch.float32) * 0.02).to(torch.float16).to(device)
        s = ql.amax_scale(w, ql.int4, block=(1, self.B))
        q = ql.quantize(w, s, ql.int4)
        self.wq = [q] + [ql.Int4Tensor(q.packed.clone(), q.shape) for _ in range(self.REPLICAS - 1)]
        self.scale = [s] + [s.clone() for _ in range(self.REPLICAS - 1)]
        self.x_host = {m: torch.randn((m, self.K), generator=g, dtype=torch.float32).to(torch.float16).pin_memory() for m in self.MS}
        self.x = {m: self.x_host[m].to(device) for m in self.MS}
        self.y = {m: torch.empty((m, self.N), dtype=torch.float16, device=device) for m in self.MS}
        self.y_host = {m: torch.empty((m, self.N), dtype=torch.float16).pin_memory() for m in self.MS}
        self.turn = 0

    def run_part(self, m):
        i = self.turn % self.REPLICAS
        self.turn += 1
        self.ql.linear_w4a16(self.x[m], self.wq[i], self.scale[i], out=self.y[m], weights_constant=True)   # quantized once, in __init__

    def parts(self):
        return [(f"M={m}", (lambda m=m: self.run_part(m)), 2 * m * self.N * self.K,
                 self.N * self.K // 2 + self.N * (self.K // self.B) * 2 + m * self.K * 2 + m * self.N * 2, "hbm") for m in self.MS]

    def e2e_units(self, step):
        # one unit per batch size: each has its own device and host buffers
        return [(("x", m), ("y", m), (lambda m=m: self.x[m].copy_(self.x_host[m], non_blocking=True)), (lambda m=m: self.run_part(m)),
                 (lambda m=m: self.y_host[m].copy_(self.y[m], non_blocking=True))) for m in self.MS]

    def e2e_bytes(self):
        return sum(m * self.K * 2 for m in self.MS), sum(m * self.N * 2 for m in self.MS)

    def config(self):
        return {"workload": self.name, "N": self.N, "K": self.K, "block": self.B, "M": list(self.MS),
                "l2": f"{self.REPLICAS} weight replicas (198 MiB > 126 MiB L2) cycled per launch", "seed": 1003}


class QdqInt8(Workload):
    """Config 1: x f32 [4096,4096] ~ N(0,1), scale = max|x|/127; one pass writes q (int8) and
    y = q*scale (f32)."""

    name = "config1_int8_qdq_round_trip"
    metric = "Q/DQ HBM GB/s (config 1: per-tensor int8 quantize + dequantize round trip, f32 [4096,4096])"
    unit = "GB/s"
    dtype = "f32 -> int8 -> f32"
    SHAPE = (4096, 4096)
    REPLICAS = 4  # 4 x (64 + 16 + 64) MiB

    def __init__(self, torch, ql, device, dist=None, seed=1001):
        self.torch, self.ql, self.device = torch, ql, device
        g = torch.Generator(device="cpu").manual_seed(seed)
        self.x_host = torch.randn(self.SHAPE, generator=g, dtype=torch.float32).pin_memory()
        x = self.x_host.to(device)
        self.scale = ql.amax_scale(x, ql.int8)
        self.x = [x] + [x.clone() for _ in range(self.REPLICAS - 1)]
        self.q = [torch.empty(self.SHAPE, dtype=torch.int8, device=device) for _ in range(self.REPLICAS)]
        self.y = [torch.empty(self.SHAPE, dtype=torch.float32, device=device) for _ in range(self.REPLICAS)]
        self.q_host = torch.empty(self.SHAPE, dtype=torch.int8).pin_memory()
        self.y_host = torch.empty(self.SHAPE, dtype=torch.float32).pin_memory()
        self.turn = 0
        from qlinear import _lib
        from qlinear.tensor import current_stream, ql_view
        self._lib, self._view, self._stream = _lib, ql_view, current_stream

    def run_part(self):
        i = self.turn % self.REPLICAS
        self.turn += 1
        L = self._lib
        tx, ts, tq, ty = self._view(self.x[i]), self._view(self.scale), self._view(self.q[i]), self._view(self.y[i])
        L.check(L.lib().ql_quantize_dequantize(tx, ts, tq, ty, L.make_attrs(), self._stream(self.device)))
        return i

    def parts(self):
        n = self.SHAPE[0] * self.SHAPE[1]
        return [("fused_qdq", self.run_part, 0, 9 * n, "hbm")]

    def e2e_units(self, step):
        i = step % self.REPLICAS   # successive steps use different device buffers; the host side is shared

        def run():
            self.turn = i
            self.run_part()

        def out():
            self.q_host.copy_(self.q[i], non_blocking=True)
            self.y_host.copy_(self.y[i], non_blocking=True)
        return [(("x", i), ("y", i), (lambda: self.x[i].copy_(self.x_host, non_blocking=True)), run, out)]

    def e2e_bytes(self):
        n = self.SHAPE[0] * self.SHAPE[1]
        return 4 * n, 5 * n

    def config(self):
        return {"workload": self.name, "shape": list(self.SHAPE), "scale": "max|x|/127 (f32, computed on the GPU)",
                "l2": f"{self.REPLICAS} input/output replicas (576 MiB > 126 MiB L2) cycled per step", "seed": 1001}


class Fp8Gemm(Workload):
    """Config 4: X bf16 [8192,8192] ~ N(0,1) quantized per step to e4m3 with scale amax/448; W [28672,8192]
    (the [8192,28672] matrix of the config held in Linear's [out,in] layout) ~ N(0,0.02) quantized once
    per tensor; Y = (Xq . Wq^T) * sx * sw, bf16.  With g GPUs each rank owns N/g output columns and the
    ranks all-gather Y (strong scaling)."""

    name = "config4_fp8_w8a8_gemm"
    metric = "quantized GEMM TFLOP/s (config 4: fp8 e4m3 W8A8, 8192x8192x28672, dynamic per-tensor activation scale)"
    unit = "TFLOP/s"
    dtype = "e4m3 x e4m3 -> f32 accumulate -> bf16"
    M, K, N = 8192, 8192, 28672
    use_graphs = False
    scaling = "strong"

    def __init__(self, torch, ql, device, dist=None, seed=1004):
        self.torch, self.ql, self.device, self.dist = torch, ql, device, dist
        self.world = dist.get_world_size() if dist is not None else 1
        self.rank = dist.get_rank() if dist is not None else 0
        self.fused = self.world > 1 and ql.peer.available() and not os.environ.get("QL_BENCH_NCCL")
        self.parallelism = (f"column-parallel over {self.world} GPUs, " +
                            ("Y [M,N] assembled on every GPU by the GEMM epilogue (multimem.st through NVSwitch), one barrier per step"
                             if self.fused else "NCCL all-gather of Y")) if self.world > 1 else "1 GPU"
        nl = self.N // self.world
        self.nl = nl
        g = torch.Generator(device="cpu").manual_seed(seed)
        self.x_host = torch.randn((self.M, self.K), generator=g, dtype=torch.float32).to(torch.bfloat16).pin_memory()
        self.x = self.x_host.to(device)
        # the weight shard of this rank, drawn from the same stream on every rank
        wq_parts, amax = [], torch.zeros((), device=device)
        gw = torch.Generator(device="cpu").manual_seed(seed + 1)
        rows = 1024
        shard = torch.empty((nl, self.K), dtype=torch.bfloat16, device=device)
        for r0 in range(0, self.N, rows):
            blk = (torch.randn((rows, self.K), generator=gw, dtype=torch.float32) * 0.02).to(torch.bfloat16)
            amax = torch.maximum(amax, blk.float().abs().max().to(device))
            lo, hi = self.rank * nl, (self.rank + 1) * nl
            if r0 + rows > lo and r0 < hi:
                a, b = max(r0, lo), min(r0 + rows, hi)
                shard[a - lo:b - lo] = blk[a - r0:b - r0].to(device)
        self.sw = (amax / 448.0).to(torch.bfloat16)            # per-tensor weight scale (rounded to the data type)
        self.wq = ql.quantize(shard, self.sw, ql.float8)
        self.sw32 = self.sw.float().reshape(())
        del shard
        self.sx32 = torch.empty((), dtype=torch.float32, device=device)
        self.xq = torch.empty((self.M, self.K), dtype=torch.float8_e4m3fn, device=device)
        self.y_local = torch.empty((self.M, nl), dtype=torch.bfloat16, device=device)
        self.y_all = torch.empty((self.world, self.M, nl), dtype=torch.bfloat16, device=device) if self.world > 1 and not self.fused else None
        # fused: two full-width outputs used in turn, so that a rank still reading step i is not overwritten by step i+1
        self.y_peer = [ql.peer.PeerTensor((self.M, self.N), torch.bfloat16) for _ in range(2)] if self.fused else None
        self.step_no = 0
        self.y_host = torch.empty((self.M, nl), dtype=torch.bfloat16).pin_memory()

    def p_scale(self):
        self.ql.amax_scale(self.x, self.ql.float8, scale_dtype=self.ql.float32, out=self.sx32)

    def p_quant(self):
        self.ql.quantize_to(self.x, self.sx32, self.xq)

    def p_gemm(self):
        self.ql.gemm_fp8(self.xq, self.wq, self.sx32, self.sw32, out=self.y_local)

    def p_gather(self):
        self.dist.all_gather_into_tensor(self.y_all, self.y_local)

    def p_gemm_store_all(self):
        self.ql.peer.gemm_fp8_peer(self.xq, self.wq, self.sx32, self.sw32, self.y_peer[self.step_no % 2], self.ql.peer.STORE_ALL,
                                   col0=self.rank * self.nl)

    def p_barrier(self):
        self.y_peer[self.step_no % 2].barrier()
        self.step_no += 1

    def parts(self):
        mk = self.M * self.K
        gemm_flops, gemm_bytes = 2 * self.M * self.K * self.nl, mk + self.nl * self.K + 2 * self.M * self.nl
        ps = [("x_amax_scale", self.p_scale, 0, 2 * mk, "hbm"), ("x_quantize", self.p_quant, 0, 3 * mk, "hbm")]
        if self.fused:
            # every rank receives the other ranks' columns while it computes: the slower of the two bounds the kernel
            ps += [("fp8_gemm_store_all", self.p_gemm_store_all, gemm_flops, gemm_bytes, "tensor_fp8"),
                   ("barrier", self.p_barrier, 0, 0, "nvlink")]
        else:
            ps.append(("fp8_gemm", self.p_gemm, gemm_flops, gemm_bytes, "tensor_fp8"))
            if self.world > 1:
                ps.append(("all_gather_y", self.p_gather, 0, 2 * self.M * self.nl * (self.world - 1), "nvlink"))
        return ps

    def step_flops_global(self):
        return 2 * self.M * self.K * self.N

    def compare(self, steps):
        """Library kernels on the same operands, same box, same run (comparison only, never the product
        path): cuBLASLt fp8 through torch._scaled_mm."""
        torch = self.torch
        out = {}
        try:
            one = torch.tensor(1.0, device=self.device)
            fn = lambda: torch._scaled_mm(self.xq, self.wq.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
            for _ in range(3):
                fn()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            for _ in range(steps):
                fn()
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / steps
            out["cublaslt_fp8_scaled_mm"] = {"ms": ms, "TFLOP/s": 2 * self.M * self.K * self.nl / ms / 1e9}
        except Exception as e:  # comparison is best effort
            out["cublaslt_fp8_scaled_mm"] = {"error": repr(e)[:200]}
        if os.environ.get("QL_BENCH_FLASHINFER"):
            # the kernel the reference reaches on Blackwell through its TVM-FFI plug-in
            # (mlir-tensorrt/integrations/PJRT/python/mlir_tensorrt_jax/flashinfer/gemm.py:85-184); slow to import, so on request
            try:
                import flashinfer
                one = torch.tensor(1.0, device=self.device)
                xf, wf = self.xq.unsqueeze(0), self.wq.unsqueeze(0).transpose(1, 2)
                o = torch.empty((1, self.M, self.nl), device=self.device, dtype=torch.bfloat16)
                fn = lambda: flashinfer.bmm_fp8(xf, wf, one, one, torch.bfloat16, o)
                for _ in range(3):
                    fn()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                a.record()
                for _ in range(steps):
                    fn()
                b.record()
                torch.cuda.synchronize()
                ms = a.elapsed_time(b) / steps
                out["flashinfer_bmm_fp8"] = {"ms": ms, "TFLOP/s": 2 * self.M * self.K * self.nl / ms / 1e9}
            except Exception as e:
                out["flashinfer_bmm_fp8"] = {"error": repr(e)[:200]}
        return out

    def e2e_units(self, step):
        def run():
            for _, fn, _, _, _ in self.parts():
                fn()

        def out():
            if self.fused:
                lo = self.rank * self.nl   # this rank reads back its share of the assembled result
                self.y_host.copy_(self.y_peer[(self.step_no - 1) % 2].local[:, lo:lo + self.nl], non_blocking=True)
            else:
                self.y_host.copy_(self.y_local, non_blocking=True)
        return [(("x", 0), ("y", 0), (lambda: self.x.copy_(self.x_host, non_blocking=True)), run, out)]

    def e2e_bytes(self):
        return self.M * self.K * 2, self.M * self.nl * 2

    def config(self):
        return {"workload": self.name, "M": self.M, "K": self.K, "N": self.N, "N_per_gpu": self.nl,
                "weights": "e4m3 per-tensor, quantized once; stored [N,K]", "activations": "bf16 -> e4m3 every step, scale = amax/448",
                "l2": "operands and output (>= 600 MiB per GPU) exceed the 126 MiB L2", "seed": 1004}


class Fp8Mlp(Workload):
    """Config 5: Llama-style MLP block, hidden 8192, intermediate 28672, 4096 tokens, bf16 activations,
    fp8 e4m3 per-output-channel gate/up/down weights ~ N(0,0.02).  RMSNorm(eps 1e-5, weight 1) fused with
    per-token fp8 quantize -> gate/up GEMM with SwiGLU in its epilogue -> per-token re-quantize -> down GEMM.
    With g GPUs: gate/up column-parallel, down row-parallel, the partial results summed over the ranks
    (strong scaling: the same block, split)."""

    name = "config5_fp8_mlp_block"
    metric = "quantized GEMM TFLOP/s (config 5: fp8 e4m3 Llama-style MLP block, 4096 tokens, 8192 -> 28672 -> 8192)"
    unit = "TFLOP/s"
    dtype = "e4m3 x e4m3 -> f32 accumulate -> bf16"
    T, H, I = 4096, 8192, 28672
    use_graphs = False
    scaling = "strong"
    PROTOCOLS = {
        "add_all": "partial sums added into both GPUs' outputs by the down-projection epilogue (multimem.red), one barrier",
        "add_owner": "partial sums added into the owner's rows by the down-projection epilogue (red over peer memory), "
                     "barrier, owners broadcast their rows (multimem.st), barrier",
        "switch_reduce": "down projection into the local copy, barrier, in-switch sum of each GPU's own rows written to all "
                         "GPUs (multimem.ld_reduce + multimem.st), barrier",
        "switch_pipelined": "down projection in token slabs into the local copy; per slab, on a side stream, barrier + in-switch sum of "
                            "each GPU's own rows written to all GPUs (multimem.ld_reduce + multimem.st) under the next slab's GEMM; "
                            "one closing barrier",
        "nccl": "NCCL all-reduce"}

    def __init__(self, torch, ql, device, dist=None, seed=1005):
        self.torch, self.ql, self.device, self.dist = torch, ql, device, dist
        self.world = dist.get_world_size() if dist is not None else 1
        self.rank = dist.get_rank() if dist is not None else 0
        fused = os.environ.get("QL_BENCH_MLP_PROTOCOL", "auto") if not os.environ.get("QL_BENCH_NCCL") else False
        il = self.I // self.world
        self.il = il
        g = torch.Generator(device=device).manual_seed(seed * 100 + self.rank)   # this rank's shard of the random weights
        def w(shape):
            return (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        self.mlp = ql.QuantizedMLP(w((il, self.H)), w((il, self.H)), w((self.H, il)), eps=1e-5, group=(dist.group.WORLD if dist is not None else None),
                                    fused_all_reduce=fused, fused_swiglu=not os.environ.get("QL_BENCH_UNFUSED_SWIGLU"))
        if os.environ.get("QL_BENCH_MLP_SLABS"):
            self.mlp.slabs = int(os.environ["QL_BENCH_MLP_SLABS"])
        gx = torch.Generator(device="cpu").manual_seed(seed)
        self.x_host = torch.randn((self.T, self.H), generator=gx, dtype=torch.float32).to(torch.bfloat16).pin_memory()
        self.x = self.x_host.to(device)
        self.x_in = [self.x, torch.empty_like(self.x)]   # end to end: the next step's upload runs under this step's kernels
        self.buf = self.mlp._buffers(self.T, device)
        proto = self.buf["protocol"]
        self.parallelism = (f"tensor-parallel over {self.world} GPUs: gate/up column-parallel, down row-parallel, " + self.PROTOCOLS[proto])
        # every rank ends with the whole result; each reads its own share of the rows back
        self.rows_out = self.T // self.world
        self.y_host = [torch.empty((self.rows_out, self.H), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        # End to end with several ranks: every rank uploads only its own T/g rows of X and the ranks complete each
        # other's copies over NVLink (a row broadcast into every replica and a barrier), instead of g full uploads
        # through one host.
        self.x_peer = None
        if self.world > 1 and proto != "nccl":
            self.x_peer = [ql.peer.PeerTensor((self.T, self.H), torch.bfloat16, dist.group.WORLD) for _ in range(2)]

    def parts(self):
        T, H, il, m, b = self.T, self.H, self.il, self.mlp, self.buf
        ps = [("rmsnorm_quant", lambda: m.stage_norm_quant(self.x, b), 0, 3 * T * H + 4 * T, "hbm")]
        if m.fused_swiglu:
            ps += [("gate_up_gemm_swiglu", lambda: m.stage_gate_up(b), 2 * T * H * 2 * il, T * H + 2 * il * H + 2 * T * il, "tensor_fp8"),
                   ("quantize_rows", lambda: m.stage_swiglu_quant(b), 0, 2 * T * il + T * il, "hbm")]
        else:
            ps += [("gate_up_gemm", lambda: m.stage_gate_up(b), 2 * T * H * 2 * il, T * H + 2 * il * H + 2 * T * 2 * il, "tensor_fp8"),
                   ("swiglu_quant", lambda: m.stage_swiglu_quant(b), 0, 2 * T * 2 * il + T * il, "hbm")]
        down = (2 * T * il * H, T * il + H * il + 2 * T * H, "tensor_fp8")
        proto = b["protocol"]
        nv_bytes = 2 * T * H                       # what crosses NVLink per GPU and direction in an all-reduce of Y, at most
        if proto == "nccl":
            ps.append(("down_gemm", lambda: m.stage_down(b)) + down)
            if self.world > 1:
                ps.append(("all_reduce_y", lambda: m.stage_all_reduce(b), 0, nv_bytes, "nvlink"))
            return ps

        def finish():
            m.stage_barrier(b)
            m._step += 1
        if proto == "switch_pipelined":
            def down_slabs():
                for s_ in range(b["slabs"]):
                    m.stage_down_slab(b, s_)

            def reduce_slabs():
                for s_ in range(b["slabs"]):
                    m.stage_reduce_slab(b, s_)
            ps += [("down_gemm_slabs", down_slabs) + down,
                   ("barrier_and_switch_reduce_slabs", reduce_slabs, 0, nv_bytes, "nvlink")]
        elif proto == "switch_reduce":
            ps += [("down_gemm", lambda: m.stage_down_local(b)) + down,
                   ("barrier_partials", lambda: m.stage_barrier(b), 0, 0, "nvlink"),
                   ("switch_reduce_owned_rows", lambda: m.stage_switch_reduce_owned(b), 0, nv_bytes, "nvlink")]
        else:
            scatter = proto == "add_owner"
            ps += [("down_gemm_add_owner" if scatter else "down_gemm_add_all", lambda: m.stage_down_add(b)) + down,
                   ("clear_next_output", lambda: m.stage_clear_next(b), 0, 2 * T * H // (self.world if scatter else 1), "hbm")]
            if scatter:
                ps += [("barrier_sums", lambda: m.stage_barrier(b), 0, 0, "nvlink"),
                       ("broadcast_owned_rows", lambda: m.stage_broadcast_owned(b), 0, 2 * T * H * (self.world - 1) // self.world, "nvlink")]
        ps.append(("barrier", finish, 0, 0, "nvlink"))
        return ps

    def run_step(self):
        return self.mlp(self.x)

    def reset(self):
        self.mlp.reset_peer_buffers()

    def step_flops_global(self):
        return 3 * 2 * self.T * self.H * self.I

    def parity_check(self):
        """The step's result against independent routes, before anything is timed.  (1) A band of tokens recomputed
        stage by stage through the plain entry points: RMSNorm+quantize, the gate/up GEMM with an f32 result, SwiGLU
        and the row maximum in torch, tensorrt.quantize per row, the down GEMM with an f32 result, partial results
        summed over the ranks by NCCL in f32.  (2) With several ranks, the whole result of the NCCL all-reduce
        variant of the block on the same shards.  (3) Every rank holds the same bits.  (4) No kernel gave up a wait."""
        import copy
        import ctypes
        torch, ql, dist, m = self.torch, self.ql, self.dist, self.mlp
        y = self.run_step().clone()
        torch.cuda.synchronize()
        # Bounds.  One rank: the benchmark's 1e-2 of the largest reference value.  Several ranks: the peer protocols and
        # NCCL add bf16 partial results rank by rank, each addition rounding to bf16 (2^-9 relative), so the worst
        # element may be off by (g - 1) more roundings of values of the output's magnitude; the error over the whole
        # band (Frobenius norm) stays far below 1e-2 and is held to that.
        bound_max = 1e-2 + (0.0025 * self.world if self.world > 1 else 0.0)
        out = {"rows_checked_stage_by_stage": 0, "bound_max_rel": bound_max, "bound_frobenius_rel": 1e-2}
        worst, worst_fro = 0.0, 0.0
        for r0 in (0, self.T - 128):
            xb = self.x[r0:r0 + 128].contiguous()
            xq, sx = ql.rmsnorm_quant_fp8(xb, 1e-5)
            gu = ql.gemm_fp8(xq, m.wq_gu, sx, m.s_gu, out_dtype=ql.float32)
            if m.fused_swiglu:
                gu = gu.reshape(128, -1, 2, 32)
                g_, u_ = gu[:, :, 0, :].reshape(128, -1), gu[:, :, 1, :].reshape(128, -1)
            else:
                gu = gu.to(torch.bfloat16).float()   # the row kernel reads the projection in the activation type
                g_, u_ = gu[:, :self.il], gu[:, self.il:]
            a = (torch.nn.functional.silu(g_) * u_)
            a = a.to(torch.bfloat16).contiguous() if m.fused_swiglu else a.contiguous()
            am = a.float().abs().amax(dim=1)
            s_a = torch.div(am, torch.full_like(am, 448.0))   # tensor / tensor: an IEEE division (a Python scalar divisor becomes a reciprocal multiply)
            s_a = torch.where(s_a == 0, torch.ones_like(s_a), s_a)
            aq = torch.empty(a.shape, dtype=torch.float8_e4m3fn, device=a.device)
            ql.quantize_to(a, s_a, aq, dim=0)
            part = ql.gemm_fp8(aq, m.wq_d, s_a, m.s_d, out_dtype=ql.float32)
            if dist is not None:
                dist.all_reduce(part)
            ref = part.double()
            diff = y[r0:r0 + 128].double() - ref
            worst = max(worst, float(diff.abs().max() / ref.abs().max().clamp_min(1e-30)))
            worst_fro = max(worst_fro, float(diff.norm() / ref.norm().clamp_min(1e-30)))
            out["rows_checked_stage_by_stage"] += 128
        out["max_rel_vs_stage_by_stage"] = worst
        out["frobenius_rel_vs_stage_by_stage"] = worst_fro
        ok = worst < bound_max and worst_fro < 1e-2
        if dist is not None and self.buf["protocol"] != "nccl":
            plain = copy.copy(m)
            plain.fused_all_reduce, plain._force, plain._buf, plain._comm = False, None, {}, None
            y2 = plain(self.x)
            e2 = float((y.double() - y2.double()).abs().max() / y2.double().abs().max().clamp_min(1e-30))
            out["max_rel_vs_nccl_all_reduce"] = e2
            ok = ok and e2 < bound_max
            del plain, y2
        if dist is not None:
            v = y.view(torch.int16).to(torch.int64)
            sig = torch.stack([v.sum(), (v * torch.arange(1, v.shape[1] + 1, device=v.device)).sum()])
            lo, hi = sig.clone(), sig.clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX)
            out["ranks_identical"] = bool(torch.equal(lo, hi))
            ok = ok and out["ranks_identical"]
        code = ctypes.c_int32(0)
        rc = ql.lib().ql_gemm_status(ctypes.byref(code))
        out["device_wait_status"] = int(code.value)
        ok = ok and rc == 0
        if dist is not None:
            t = torch.tensor([1.0 if ok else 0.0, out["max_rel_vs_stage_by_stage"], out["frobenius_rel_vs_stage_by_stage"]], device=self.device,
                             dtype=torch.float64)
            agree, worst_all = t[:1].clone(), t[1:].clone()
            dist.all_reduce(agree, op=dist.ReduceOp.MIN)
            dist.all_reduce(worst_all, op=dist.ReduceOp.MAX)
            ok = bool(agree.item() > 0.5)
            out["max_rel_vs_stage_by_stage"], out["frobenius_rel_vs_stage_by_stage"] = float(worst_all[0]), float(worst_all[1])
        out["max_rel"] = max(out["max_rel_vs_stage_by_stage"], out.get("max_rel_vs_nccl_all_reduce", 0.0))
        out["ok"] = bool(ok)
        self.reset()
        return out

    def compare(self, steps):
        """Library kernel on the gate/up projection's operands, same box, same process (comparison only, never the
        product path): cuBLASLt fp8 through torch._scaled_mm, per-tensor scales, bf16 result."""
        torch = self.torch
        out = {}
        try:
            b = self.buf
            one = torch.tensor(1.0, device=self.device)
            fn = lambda: torch._scaled_mm(b["xq"], self.mlp.wq_gu.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
            for _ in range(3):
                fn()
            a_, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a_.record()
            for _ in range(steps):
                fn()
            b_.record()
            torch.cuda.synchronize()
            ms = a_.elapsed_time(b_) / steps
            out["cublaslt_fp8_gate_up_shape"] = {"ms": ms, "TFLOP/s": 2 * self.T * self.H * 2 * self.il / ms / 1e9}
        except Exception as e:  # comparison is best effort
            out["cublaslt_fp8_gate_up_shape"] = {"error": repr(e)[:200]}
        return out

    def e2e_units(self, step):
        # two input buffers and the block's two result buffers, used in turn: step i+1 is uploaded while step i runs
        # and step i's result is read back while step i+1 runs
        box, k = {}, step % 2
        ko = k   # every protocol leaves a result intact during the next call

        r0 = self.rank * self.rows_out

        def out():
            self.y_host[k].copy_(box["y"][r0:r0 + self.rows_out], non_blocking=True)
        if self.x_peer is not None:
            xp = self.x_peer[k]

            def run_shared():
                xp.broadcast_rows(r0, self.rows_out)   # my rows into every rank's copy of X
                xp.barrier()                           # ... and everybody else's into mine
                box["y"] = self.mlp(xp.local)
            return [(("x", k), ("y", ko), (lambda: xp.local[r0:r0 + self.rows_out].copy_(self.x_host[r0:r0 + self.rows_out], non_blocking=True)),
                     run_shared, out)]

        def run():
            box["y"] = self.mlp(self.x_in[k])
        return [(("x", k), ("y", ko), (lambda: self.x_in[k].copy_(self.x_host, non_blocking=True)), run, out)]

    def e2e_bytes(self):
        # whole job: every row of X goes up once (in g pieces) unless each rank uploads all of it; every row of Y comes down once
        up = self.T * self.H * 2 * (1 if (self.x_peer is not None or self.world == 1) else self.world)
        return up, self.T * self.H * 2

    def config(self):
        return {"workload": self.name, "tokens": self.T, "hidden": self.H, "intermediate": self.I, "intermediate_per_gpu": self.il,
                "weights": "e4m3 per output channel, quantized once", "activations": "per-token e4m3, scale = row amax/448",
                "l2": "weights and activations (>= 150 MiB per GPU) exceed the 126 MiB L2", "seed": 1005}


class Nvfp4Qdq(Workload):
    """Not a BASELINE config: tensorrt.dynamic_quantize (NVFP4, blocks of 16, e4m3 block scales) of x bf16 [8192,8192]
    ~ N(0,1) and the inverse, timed as two parts."""

    name = "nvfp4_dynamic_quantize_round_trip"
    metric = "Q/DQ HBM GB/s (NVFP4 dynamic quantize + dequantize, bf16 [8192,8192])"
    unit = "GB/s"
    dtype = "bf16 -> e2m1 + e4m3 block scales -> bf16"
    SHAPE = (8192, 8192)
    REPLICAS = 3  # 3 x (128 + 32 + 4 + 128) MiB

    def __init__(self, torch, ql, device, dist=None, seed=1006):
        self.torch, self.ql, self.device = torch, ql, device
        g = torch.Generator(device="cpu").manual_seed(seed)
        self.x_host = torch.randn(self.SHAPE, generator=g, dtype=torch.float32).to(torch.bfloat16).pin_memory()
        x = self.x_host.to(device)
        n = self.SHAPE[0] * self.SHAPE[1]
        self.gs = torch.ones((), dtype=torch.float32, device=device)
        self.x = [x] + [x.clone() for _ in range(self.REPLICAS - 1)]
        self.q = [ql.Float4Tensor(torch.empty(n // 2, dtype=torch.uint8, device=device), self.SHAPE) for _ in range(self.REPLICAS)]
        self.s = [torch.empty((self.SHAPE[0], self.SHAPE[1] // 16), dtype=torch.float8_e4m3fn, device=device) for _ in range(self.REPLICAS)]
        self.y = [torch.empty(self.SHAPE, dtype=torch.bfloat16, device=device) for _ in range(self.REPLICAS)]
        self.y_host = torch.empty(self.SHAPE, dtype=torch.bfloat16).pin_memory()
        self.turn = 0
        from qlinear import _lib
        from qlinear.tensor import current_stream, ql_view
        self._lib, self._view, self._stream = _lib, ql_view, current_stream

    def p_quant(self):
        i = self.turn % self.REPLICAS
        L = self._lib
        L.check(L.lib().ql_dynamic_quantize(self._view(self.x[i]), self._view(self.gs), 1, 16, self._view(self.q[i]), self._view(self.s[i]),
                                            self._stream(self.device)))

    def p_dequant(self):
        i = self.turn % self.REPLICAS
        self.turn += 1
        L = self._lib
        L.check(L.lib().ql_dequantize_nvfp4(self._view(self.q[i]), self._view(self.s[i]), self._view(self.gs), self._view(self.y[i]),
                                            self._stream(self.device)))

    def parts(self):
        n = self.SHAPE[0] * self.SHAPE[1]
        packed = n // 2 + n // 16
        return [("dynamic_quantize", self.p_quant, 0, 2 * n + packed, "hbm"), ("dequantize", self.p_dequant, 0, packed + 2 * n, "hbm")]

    def e2e_units(self, step):
        i = step % self.REPLICAS

        def run():
            self.turn = i
            self.p_quant()
            self.p_dequant()
        return [(("x", i), ("y", i), (lambda: self.x[i].copy_(self.x_host, non_blocking=True)), run,
                 (lambda: self.y_host.copy_(self.y[i], non_blocking=True)))]

    def e2e_bytes(self):
        n = self.SHAPE[0] * self.SHAPE[1]
        return 2 * n, 2 * n

    def config(self):
        return {"workload": self.name, "shape": list(self.SHAPE), "double_quant_scale": 1.0, "block": 16,
                "l2": f"{self.REPLICAS} input/output replicas (876 MiB > 126 MiB L2) cycled per step", "seed": 1006}


class Nvfp4Gemm(Workload):
    """Not a BASELINE config: the block-scaled NVFP4 GEMM on config 4's shape.  X bf16 [8192,8192] ~ N(0,1) goes through
    tensorrt.dynamic_quantize every step; W [28672,8192] ~ N(0,0.02) was quantized once; Y = dq(Xq) . dq(Wq)^T, bf16."""

    name = "nvfp4_block_scaled_gemm"
    metric = "quantized GEMM TFLOP/s (NVFP4 block-scaled GEMM, 8192x8192x28672, activations quantized every step)"
    unit = "TFLOP/s"
    dtype = "e2m1 x e2m1, e4m3 block scales -> f32 accumulate -> bf16"
    M, K, N = 8192, 8192, 28672
    use_graphs = False

    def __init__(self, torch, ql, device, dist=None, seed=1007):
        self.torch, self.ql, self.device = torch, ql, device
        g = torch.Generator(device="cpu").manual_seed(seed)
        self.x_host = torch.randn((self.M, self.K), generator=g, dtype=torch.float32).to(torch.bfloat16).pin_memory()
        self.x = self.x_host.to(device)
        wq, ws = [], []
        for r0 in range(0, self.N, 4096):
            blk = (torch.randn((4096, self.K), generator=g, dtype=torch.float32) * 0.02).to(torch.bfloat16).to(device)
            d, sc = ql.dynamic_quantize(blk, 1.0)
            wq.append(d.packed)
            ws.append(sc)
        self.wq = ql.Float4Tensor(torch.cat(wq), (self.N, self.K))
        self.ws = torch.cat(ws, dim=0).contiguous()
        self.xq, self.xs = ql.dynamic_quantize(self.x, 1.0)
        self.y = torch.empty((self.M, self.N), dtype=torch.bfloat16, device=device)
        self.y_host = torch.empty((self.M, self.N), dtype=torch.bfloat16).pin_memory()
        from qlinear import _lib
        from qlinear.tensor import current_stream, ql_view
        self._lib, self._view, self._stream = _lib, ql_view, current_stream
        self.gs = torch.ones((), dtype=torch.float32, device=device)

    def p_quant(self):
        L = self._lib
        L.check(L.lib().ql_dynamic_quantize(self._view(self.x), self._view(self.gs), 1, 16, self._view(self.xq), self._view(self.xs), self._stream(self.device)))

    def p_gemm(self):
        self.ql.gemm_nvfp4(self.xq, self.xs, self.wq, self.ws, out=self.y)

    def parts(self):
        M, K, N = self.M, self.K, self.N
        n = M * K
        return [("dynamic_quantize_x", self.p_quant, 0, 2 * n + n // 2 + n // 16, "hbm"),
                ("nvfp4_gemm", self.p_gemm, 2 * M * N * K, (M + N) * (K // 2 + K // 16) + 2 * M * N, "tensor_fp4")]

    def e2e_units(self, step):
        def run():
            self.p_quant()
            self.p_gemm()
        return [(("x", 0), ("y", 0), (lambda: self.x.copy_(self.x_host, non_blocking=True)), run,
                 (lambda: self.y_host.copy_(self.y, non_blocking=True)))]

    def e2e_bytes(self):
        return 2 * self.M * self.K, 2 * self.M * self.N

    def config(self):
        return {"workload": self.name, "M": self.M, "K": self.K, "N": self.N, "block": 16, "double_quant_scale": 1.0,
                "l2": "operands and output (>= 600 MiB) exceed the 126 MiB L2", "seed": 1007}


WORKLOADS = {"nvfp4gemm": Nvfp4Gemm, "c1": QdqInt8, "c2": W8A16Linear, "c3": W4A16Linear, "c4": Fp8Gemm, "c5": Fp8Mlp, "nvfp4": Nvfp4Qdq}


# ----------------------------------------------------------------------------------------------
# the reference arm and the CPU baseline: oracle/ on the host cores, bounded sample
# ----------------------------------------------------------------------------------------------
def cpu_reference(workload: str, budget_s: float = 12.0):
    """Times the CPU restatement of the reference's host path (oracle/ql_oracle.c, OpenMP over all
    host threads) on a bounded sample of the workload.  Returns (value, unit, cores, sample)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import numpy as np
    import oracle as orc
    orc.build()
    cores = orc.lib().orc_num_threads()
    rng = np.random.default_rng(7)
    if workload == "c2":
        N, K = 11008, 4096
        n_s, m_s = 256, 16
        x = orc.from_f32(rng.standard_normal((m_s, K)).astype(np.float32), orc.BF16)
        wq = rng.integers(-127, 128, size=(n_s, K), dtype=np.int8)
        s = (rng.random(n_s).astype(np.float32) * 1e-3 + 1e-4).astype(np.float16)
        t0 = time.perf_counter()
        orc.linear_w8(x, orc.BF16, wq, s, orc.F16, orc.BF16, acc64=False)
        t1 = time.perf_counter() - t0
        # grow the slice of output channels, then the rows, so that the sample takes about `budget_s`
        grow = budget_s / max(t1, 1e-4)
        n_big = int(min(N, max(n_s, n_s * grow)))
        m_s = int(min(2048, max(m_s, m_s * grow * n_s / n_big)))
        x = orc.from_f32(rng.standard_normal((m_s, K)).astype(np.float32), orc.BF16)
        wq = rng.integers(-127, 128, size=(n_big, K), dtype=np.int8)
        s = (rng.random(n_big).astype(np.float32) * 1e-3 + 1e-4).astype(np.float16)
        t0 = time.perf_counter()
        orc.linear_w8(x, orc.BF16, wq, s, orc.F16, orc.BF16, acc64=False)
        dt = time.perf_counter() - t0
        flops = 2.0 * m_s * n_big * K
        return flops / dt / 1e12, "TFLOP/s", cores, f"M={m_s} rows x {n_big} of {N} output channels x K={K}, f32 accumulation, {dt:.1f} s"
    if workload == "c3":
        N, K, B = 4096, 4096, 128
        m_s, n_s = 8, 128
        x = rng.standard_normal((m_s, K)).astype(np.float16)
        def sample(n_rows):
            wp = rng.integers(0, 256, size=(n_rows, K // 2), dtype=np.uint8)
            sc = (rng.random((n_rows, K // B)).astype(np.float32) * 1e-3 + 1e-4).astype(np.float16)
            t0 = time.perf_counter()
            orc.linear_w4(x, orc.F16, wp, sc, orc.F16, orc.F16, B, acc64=False)
            return time.perf_counter() - t0
        t1 = sample(n_s)
        n_big = int(min(N, max(n_s, n_s * budget_s / max(t1, 1e-4))))
        dt = sample(n_big)
        return 2.0 * m_s * n_big * K / dt / 1e12, "TFLOP/s", cores, f"M={m_s} rows x {n_big} of {N} output channels x K={K}, block {B}, f32 accumulation, {dt:.1f} s"
    if workload == "c4":
        M, K, N = 8192, 8192, 28672
        m_s, n_s = 32, 64
        def sample(mm, nn):
            xq = rng.integers(0, 0x7F, size=(mm, K), dtype=np.uint8)
            wq = rng.integers(0, 0x7F, size=(nn, K), dtype=np.uint8)
            t0 = time.perf_counter()
            orc.gemm_fp8(xq, wq, np.float32(0.01), np.float32(0.01), orc.BF16, acc64=False)
            return time.perf_counter() - t0
        t1 = sample(m_s, n_s)
        grow = (budget_s / max(t1, 1e-4)) ** 0.5
        mm, nn = int(min(M, max(m_s, m_s * grow))), int(min(N, max(n_s, n_s * grow)))
        dt = sample(mm, nn)
        return 2.0 * mm * nn * K / dt / 1e12, "TFLOP/s", cores, f"{mm} of {M} rows x {nn} of {N} columns x K={K}, f32 accumulation, {dt:.1f} s"
    if workload == "c5":
        T, H, I = 4096, 8192, 28672
        t_s, i_s = 16, 128
        def sample(tt, ii):
            x = orc.from_f32(rng.standard_normal((tt, H)).astype(np.float32), orc.BF16)
            wgu = rng.integers(0, 0x70, size=(2 * ii, H), dtype=np.uint8)
            wd = rng.integers(0, 0x70, size=(H, ii), dtype=np.uint8)
            sgu = np.full(2 * ii, 1e-3, dtype=np.float32)
            sd = np.full(H, 1e-3, dtype=np.float32)
            t0 = time.perf_counter()
            xq, sx = orc.rmsnorm_quant_fp8(x, orc.BF16, 1e-5)
            gu = orc.gemm_fp8(xq, wgu, sx, sgu, orc.BF16, acc64=False)
            aq, sa = orc.swiglu_quant_fp8(gu, orc.BF16)
            orc.gemm_fp8(aq, wd, sa, sd, orc.BF16, acc64=False)
            return time.perf_counter() - t0
        t1 = sample(t_s, i_s)
        grow = (budget_s / max(t1, 1e-4)) ** 0.5
        tt, ii = int(min(T, max(t_s, t_s * grow))), int(min(I, max(i_s, i_s * grow)))
        dt = sample(tt, ii)
        return 3 * 2.0 * tt * H * ii / dt / 1e12, "TFLOP/s", cores, f"{tt} of {T} tokens x {ii} of {I} intermediate columns, hidden {H}, f32 accumulation, {dt:.1f} s"
    if workload == "c1":
        n = 1 << 22
        x = rng.standard_normal(n).astype(np.float32)
        s = np.array(np.abs(x).max() / 127.0, dtype=np.float32)
        reps = 0
        t0 = time.perf_counter()
        while time.perf_counter() - t0 < budget_s:
            q = orc.quantize(x, orc.F32, s, orc.F32, orc.I8)
            orc.dequantize(q, orc.I8, s, orc.F32, orc.F32, (n,))
            reps += 1
        dt = time.perf_counter() - t0
        return 9.0 * n * reps / dt / 1e9, "GB/s", 1, f"{reps} x (quantize + dequantize) of {n} f32 elements, scalar loop, {dt:.1f} s"
    if workload == "nvfp4":
        rows, K = 512, 8192
        x = orc.from_f32(rng.standard_normal((rows, K)).astype(np.float32), orc.BF16)
        reps = 0
        t0 = time.perf_counter()
        while time.perf_counter() - t0 < budget_s:
            q, sc = orc.dynamic_quantize_nvfp4(x, orc.BF16, 1.0)
            orc.dequantize_nvfp4(q, sc, 1.0, orc.BF16)
            reps += 1
        dt = time.perf_counter() - t0
        n = rows * K
        return (2 * n + n // 2 + n // 16) * 2.0 * reps / dt / 1e9, "GB/s", cores, f"{reps} x (dynamic_quantize + dequantize) of {rows} x {K} bf16 elements, {dt:.1f} s"
    if workload == "nvfp4gemm":
        K = 8192
        def sample(mm, nn):
            a = orc.from_f32(rng.standard_normal((mm, K)).astype(np.float32), orc.BF16)
            b = orc.from_f32((rng.standard_normal((nn, K)) * 0.02).astype(np.float32), orc.BF16)
            t0 = time.perf_counter()
            qa, sa = orc.dynamic_quantize_nvfp4(a, orc.BF16, 1.0)
            qb, sb = orc.dynamic_quantize_nvfp4(b, orc.BF16, 1.0)
            orc.matmul(orc.dequantize_nvfp4(qa, sa, 1.0, orc.F32), np.ascontiguousarray(orc.dequantize_nvfp4(qb, sb, 1.0, orc.F32).T), orc.F32)
            return time.perf_counter() - t0
        t1 = sample(32, 64)
        grow = (budget_s / max(t1, 1e-4)) ** 0.5
        mm, nn = int(min(8192, max(32, 32 * grow))), int(min(28672, max(64, 64 * grow)))
        dt = sample(mm, nn)
        return 2.0 * mm * nn * K / dt / 1e12, "TFLOP/s", cores, f"{mm} of 8192 rows x {nn} of 28672 columns x K={K}: dynamic_quantize, dequantize, f32 product, {dt:.1f} s"
    raise SystemExit(f"no CPU restatement for workload {workload}")


def reference_config(wl, gpus):
    """The workload's `config` object without a GPU: the same keys the product arm prints."""
    obj = object.__new__(wl)
    if hasattr(wl, "N"):
        obj.nl = wl.N // max(1, gpus)
    if hasattr(wl, "I"):
        obj.il = wl.I // max(1, gpus)
    try:
        return wl.config(obj)
    except AttributeError:
        return {"workload": wl.name}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # torchrun pins OMP_NUM_THREADS=1 for its children; this arm is meant to use every host thread
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    wl = WORKLOADS[args.workload]
    vals = []
    sample = ""
    t0 = time.perf_counter()
    per = max(2.0, min(12.0, 100.0 / max(1, args.steps + args.warmup)))
    for i in range(args.warmup + args.steps):
        v, unit, cores, sample = cpu_reference(args.workload, budget_s=per)
        if i >= args.warmup:
            vals.append(v)
    value = sum(vals) / len(vals)
    ms = (time.perf_counter() - t0) * 1e3 / (args.steps + args.warmup)
    line = {"impl": "reference", "metric": wl.metric, "value": value, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": wl.scaling, "vs_baseline": None,
            "dtype": wl.dtype, "data": "synthetic (seeded)",
            "config": dict(reference_config(wl, args.gpus), parallelism=f"{cores} host threads (OpenMP)", timing="wall clock",
                           arm="CPU restatement of the reference's host path (oracle/ql_oracle.c); the reference itself cannot "
                               "be built here"),
            "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
# the product arm
# ----------------------------------------------------------------------------------------------
def bind_to_gpu_numa_node(torch, local):
    """Best effort: run this rank's host threads on the CPUs of the NUMA node its GPU hangs off, before any pinned
    staging buffer is allocated (first touch then places the buffer on that node).  Reads sysfs only."""
    info = {"bound": False}
    try:
        pr = torch.cuda.get_device_properties(local)
        dev = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{dev}/numa_node") as f:
            node = int(f.read().strip())
        info["gpu_numa_node"] = node
        if node < 0:
            return info
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0)
        use = cpus & allowed
        info["allowed_cpus"] = len(allowed)
        if use and use != allowed:
            os.sched_setaffinity(0, use)
            info["bound"] = True
        info["cpus_on_node"] = len(use)
    except Exception as e:  # topology unreadable: leave the affinity alone
        info["error"] = repr(e)[:120]
    return info


def time_parts(torch, L, wl, parts, K, device, barrier):
    """Each part on its own: K launches back to back (captured graphs, one launch per buffer rotation, where the
    workload asks for graphs), CUDA events on the launching stream.  Returns milliseconds per launch."""
    stream = torch.cuda.current_stream(device)
    rot = getattr(wl, "REPLICAS", 1)
    part_ms = []
    for name, fn, _, _, bound in parts:
        a_, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        if wl.use_graphs:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for _ in range(rot):
                    fn()
            stream = torch.cuda.current_stream(device)
            reps = max(1, (K + rot - 1) // rot)
            g.replay()
            barrier()
            a_.record(stream)
            for _ in range(reps):
                g.replay()
            b_.record(stream)
            barrier()
            part_ms.append(a_.elapsed_time(b_) / (reps * rot))
        else:
            a_.record(stream)
            for _ in range(K):
                fn()
            b_.record(stream)
            barrier()
            ms = a_.elapsed_time(b_) / K
            if bound == "hbm" and ms < 0.3:
                # A streaming kernel of tens of microseconds launched from Python is timed by the launch path, not by
                # the device: the same K launches again as one captured graph (local kernels only).
                try:
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g):
                        for _ in range(K):
                            fn()
                    stream = torch.cuda.current_stream(device)
                    g.replay()
                    barrier()
                    a_.record(stream)
                    g.replay()
                    b_.record(stream)
                    barrier()
                    ms = min(ms, a_.elapsed_time(b_) / K)
                except Exception as exc:  # keep the directly launched figure
                    print(f"part {name}: graph capture failed ({exc}); timed by direct launches", file=sys.stderr, flush=True)
                    torch.cuda.synchronize()
            part_ms.append(ms)
    return part_ms


def peak_of(bound, peaks, lib_fp8=None):
    """(bound name for the roofline object, peak, unit, where the peak comes from).  Parts are timed alone, a few
    dozen launches back to back, so tensor-core parts are held against the burst figure."""
    if bound == "tensor":
        return "tensor", peaks["bf16_tflops"], "TFLOP/s", "measured cuBLAS bf16, burst"
    if bound == "tensor_fp8":
        note = "2 x measured cuBLAS bf16 burst (no fp8 peak is measured by the driver)"
        if lib_fp8:
            note += f"; cuBLASLt fp8 on the same operands in this process: {lib_fp8:.0f} TFLOP/s"
        return "tensor", 2 * peaks["bf16_tflops"], "TFLOP/s", note
    if bound == "tensor_fp4":
        return "tensor", 4 * peaks["bf16_tflops"], "TFLOP/s", "4 x measured cuBLAS bf16 burst (no fp4 peak is measured by the driver)"
    if bound == "nvlink":
        return "nvlink", 770.0, "GB/s", "peer copy per direction measured on this pool (900 nominal)"
    return "hbm", peaks["hbm_gbs"], "GB/s", "measured copy bandwidth"


def part_table(parts, part_ms, peaks):
    out = {}
    for (nm, _, f, b, bd), ms in zip(parts, part_ms):
        sec = ms * 1e-3
        _, peak, unit, _ = peak_of(bd, peaks)
        ach = (f / sec / 1e12) if unit == "TFLOP/s" else (b / sec / 1e9)
        out[nm] = {"ms": ms, "GB/s": b / sec / 1e9, "TFLOP/s": f / sec / 1e12, "bound": bd, "frac": ach / peak if (f or b) else None}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c5", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra-parts", action="store_true", help="skip the config 1 / config 4 kernels added to `parts` at one GPU")
    ap.add_argument("--compare", action="store_true", help="also time library kernels on the same operands (comparison only)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3

    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch
    import qlinear as ql

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    numa = bind_to_gpu_numa_node(torch, local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    wl = WORKLOADS[args.workload](torch, ql, device, dist)
    parts = wl.parts()
    stream = torch.cuda.current_stream(device)
    L = ql.lib()
    K = args.steps

    # -------- the result is checked before anything is timed
    parity = None
    if hasattr(wl, "parity_check"):
        parity = wl.parity_check()
        if not parity["ok"]:
            if rank == 0:
                print(json.dumps({"metric": wl.metric, "parity_check": parity, "error": "the step's result failed its parity check; nothing was timed"}),
                      flush=True)
            if dist is not None:
                dist.destroy_process_group()
            raise SystemExit(3)

    def run_step():
        if hasattr(wl, "run_step"):
            wl.run_step()
        else:
            for _, fn, _, _, _ in parts:
                fn()

    for _ in range(args.warmup):
        run_step()
    barrier()

    # Optionally replay captured CUDA graphs, so that what is timed is the device work and not the
    # Python/ctypes launch path.  One graph per buffer rotation keeps every launch on cold data.
    rot = getattr(wl, "REPLICAS", 1)
    step_graphs, launches_per_step = None, None
    if wl.use_graphs:
        step_graphs = []
        for _ in range(rot):
            g = torch.cuda.CUDAGraph()
            c0 = L.ql_launch_count()
            with torch.cuda.graph(g):
                run_step()
            launches_per_step = L.ql_launch_count() - c0
            step_graphs.append(g)
        stream = torch.cuda.current_stream(device)
        for g in step_graphs:  # one untimed replay each
            g.replay()
        barrier()

    clocks = ClockSampler(local)
    clocks.start()
    clocks.wait_ready()

    # -------- whole steps, device-resident inputs
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = L.ql_launch_count()
    barrier()
    t_start.record(stream)
    for s_ in range(K):
        if step_graphs:
            step_graphs[s_ % rot].replay()
        else:
            run_step()
    t_end.record(stream)
    barrier()
    total_ms = t_start.elapsed_time(t_end)
    launches = (launches_per_step * K) if step_graphs else (L.ql_launch_count() - launches0)

    # -------- each part on its own: the roofline numbers
    if hasattr(wl, "reset"):
        wl.reset()
    part_ms = time_parts(torch, L, wl, parts, K, device, barrier)
    comparison = wl.compare(K) if hasattr(wl, "compare") and (args.compare or args.workload == "c5") else None
    clock_info = clocks.stop()

    # -------- end to end: inputs from pinned host memory, results read back, every step.  Copies in, kernels and
    # copies out run on three streams; a unit of work (one input buffer, one output buffer) is chained by events,
    # so that a step's read-back overlaps the next step's upload and kernels wherever the buffers allow it.
    if hasattr(wl, "reset"):
        wl.reset()   # the per-part loops above ran stages out of turn
    s_in, s_run, s_out = torch.cuda.Stream(device), stream, torch.cuda.Stream(device)
    run_done, in_ready, out_done = {}, {}, {}

    stage_events = []   # per timed unit: (upload start, upload end, kernels start, kernels end, read-back start, read-back end)

    def e2e_step(step, timed=False):
        def mark(st):
            e = torch.cuda.Event(enable_timing=True)
            e.record(st)
            return e
        for in_key, out_key, f_in, f_run, f_out in wl.e2e_units(step):
            with torch.cuda.stream(s_in):
                if in_key in run_done:
                    s_in.wait_event(run_done[in_key])      # the previous user of this input buffer has read it
                t0 = mark(s_in) if timed else None
                f_in()
                in_ready[in_key] = t1 = mark(s_in)
            with torch.cuda.stream(s_run):
                s_run.wait_event(in_ready[in_key])
                if out_key in out_done:
                    s_run.wait_event(out_done[out_key])    # the previous result in this output buffer has been read back
                t2 = mark(s_run) if timed else None
                f_run()
                ev = mark(s_run)
                run_done[in_key] = ev
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev)
                t4 = mark(s_out) if timed else None
                f_out()
                out_done[out_key] = t5 = mark(s_out)
            if timed:
                stage_events.append((t0, t1, t2, ev, t4, t5))

    def e2e_join():
        stream.wait_stream(s_in)
        stream.wait_stream(s_out)

    for i in range(3):
        e2e_step(i)
    e2e_join()
    barrier()
    e_start, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_start.record(stream)
    s_in.wait_stream(stream)
    s_out.wait_stream(stream)
    for i in range(K):
        e2e_step(3 + i, timed=True)
    e2e_join()
    e_end.record(stream)
    barrier()
    e2e_ms = e_start.elapsed_time(e_end)
    # where an end-to-end step spends its time on this rank: mean device time of each stage, and the mean distance between
    # the starts of consecutive steps' kernels (the steady-state period)
    n_ev = max(1, len(stage_events))
    e2e_stages = {"upload_ms": sum(a.elapsed_time(b) for a, b, _, _, _, _ in stage_events) / n_ev,
                  "kernels_ms": sum(c.elapsed_time(d) for _, _, c, d, _, _ in stage_events) / n_ev,
                  "read_back_ms": sum(e.elapsed_time(f) for _, _, _, _, e, f in stage_events) / n_ev,
                  "kernels_wait_for_upload_ms": sum(max(0.0, p[3].elapsed_time(q[2])) for p, q in zip(stage_events, stage_events[1:])) / max(1, n_ev - 1)}

    if dist is not None:
        st_keys = sorted(e2e_stages)
        st = torch.tensor([e2e_stages[k_] for k_ in st_keys], device=device, dtype=torch.float64)
        dist.all_reduce(st, op=dist.ReduceOp.MAX)
        e2e_stages = {k_: float(v) for k_, v in zip(st_keys, st)}   # the slowest rank's figure for each stage
        t = torch.tensor([total_ms, e2e_ms] + part_ms, device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, e2e_ms, part_ms = float(t[0]), float(t[1]), [float(v) for v in t[2:]]

    if hasattr(wl, "step_flops_global"):
        work = wl.step_flops_global()                      # whole job, however many GPUs share it
    else:
        work = sum((f if wl.unit == "TFLOP/s" else b) for _, _, f, b, _ in parts) * world   # replicas
    denom = 1e12 if wl.unit == "TFLOP/s" else 1e9
    value = work * K / (total_ms * 1e-3) / denom
    e2e_value = work * K / (e2e_ms * 1e-3) / denom

    peaks = measured_peaks()
    lib_fp8 = None
    if comparison:
        for v in comparison.values():
            if isinstance(v, dict) and "TFLOP/s" in v:
                lib_fp8 = v["TFLOP/s"]
    dom = max(range(len(parts)), key=lambda p: part_ms[p])
    name, _, f, b, bound = parts[dom]
    sec = part_ms[dom] * 1e-3
    rb, peak, unit, note = peak_of(bound, peaks, lib_fp8)
    achieved = (f / sec / 1e12) if unit == "TFLOP/s" else (b / sec / 1e9)
    roofline = {"kernel": f"{wl.name}:{name}", "bound": rb, "achieved": achieved, "peak": peak, "unit": unit,
                "frac": achieved / peak, "peak_source": f"{peaks['source']}: {note}", "traffic": TRAFFIC.get(f"{wl.name}:{name}"),
                "algorithmic_bytes_per_launch": b, "algorithmic_flops_per_launch": f, "avg_launch_ms": part_ms[dom]}
    if lib_fp8 and bound == "tensor_fp8":
        roofline["frac_of_cublaslt_fp8"] = achieved / lib_fp8
    per_part = part_table(parts, part_ms, peaks)

    # -------- one GPU: the other two kinds of kernel of the path, timed the same way, as further entries of `parts`
    if world == 1 and args.workload == "c5" and not args.no_extra_parts:
        del wl.mlp, wl.buf
        torch.cuda.empty_cache()
        for key in ("c1", "c4"):
            w2 = WORKLOADS[key](torch, ql, device, None)
            p2 = w2.parts()
            for _ in range(3):
                for _, fn, _, _, _ in p2:
                    fn()
            ms2 = time_parts(torch, L, w2, p2, K, device, barrier)
            for nm, row in part_table(p2, ms2, peaks).items():
                row["traffic"] = TRAFFIC.get(f"{w2.name}:{nm}")
                per_part[f"{w2.name}:{nm}"] = row
            if key == "c4":
                cmp4 = w2.compare(K)
                lib4 = cmp4.get("cublaslt_fp8_scaled_mm", {}).get("TFLOP/s")
                if lib4:
                    per_part[f"{w2.name}:fp8_gemm"]["frac_of_cublaslt_fp8"] = per_part[f"{w2.name}:fp8_gemm"]["TFLOP/s"] / lib4
                    comparison = dict(comparison or {}, cublaslt_fp8_config4_shape=cmp4["cublaslt_fp8_scaled_mm"])
            del w2, p2
            torch.cuda.empty_cache()

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    h2d, d2h = wl.e2e_bytes()
    line = {"metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world, "steps": K, "warmup": args.warmup,
            "ms_per_step": total_ms / K, "higher_is_better": True, "scaling": wl.scaling, "vs_baseline": None,
            "dtype": wl.dtype, "data": "synthetic (seeded)",
            "config": dict(wl.config(), parallelism=(wl.parallelism if world > 1 else "1 GPU"),
                           timing="CUDA graph replay" if step_graphs else "direct launches"),
            "clocks": clock_info, "gpu_launches": int(launches),
            "e2e": {"value": e2e_value, "unit": wl.unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / K,
                    "overlap": "uploads, kernels and read-backs on three streams, chained per buffer by events", "host_numa": numa,
                    "stages_max_over_ranks": e2e_stages},
            "roofline": roofline, "parts": per_part}
    if parity is not None:
        line["parity_check"] = parity
    if comparison:
        line["comparison"] = comparison
    if not args.no_cpu_baseline and world == 1:
        v, u, cores, sample = cpu_reference(args.workload)
        line["cpu_baseline"] = {"value": v, "unit": u, "cores": cores, "kind": "port", "sample": sample}
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
