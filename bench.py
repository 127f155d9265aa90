#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1|c2|c3|c4] [--impl reference]

One JSON line on stdout (rank 0).  A step is one pass of the workload over one batch of seeded
synthetic input already resident in HBM; `value` is device-timed throughput over exactly K steps,
`e2e` the same metric with the step's inputs copied from pinned host memory and its results read
back inside the timed region.  Default workload: benchmark config 2 (per-channel int8 weights,
W8A16 linear, M in {1, 16, 128, 2048}); the other configs are selectable and are otherwise
covered by the parity tests.

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

    def __init__(self, index: int, period_s: float = 0.004):
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

    parts(): list of (name, fn, flops, bytes) -- the kernels of one step, each timed separately
    so that the dominant one can be reported against its roofline."""

    name = ""
    metric = ""
    unit = ""
    dtype = ""


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

    def __init__(self, torch, ql, device, seed=1002):
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
        self.ql.linear_w8a16(self.x[m], w, self.scale, out=self.y[m])

    def parts(self):
        return [(f"M={m}", (lambda m=m: self.run_part(m)), self.flops(m), self.bytes(m)) for m in self.MS]

    def e2e_step(self):
        for m in self.MS:
            self.x[m].copy_(self.x_host[m], non_blocking=True)
            self.run_part(m)
            self.y_host[m].copy_(self.y[m], non_blocking=True)

    def e2e_bytes(self):
        h2d = sum(m * self.K * 2 for m in self.MS)
        d2h = sum(m * self.N * 2 for m in self.MS)
        return h2d, d2h

    def config(self):
        return {"workload": self.name, "N": self.N, "K": self.K, "M": list(self.MS), "weights": "int8 per-channel (axis 0), f16 scales",
                "l2": f"{self.REPLICAS} weight replicas ({self.REPLICAS * self.N * self.K >> 20} MiB > 126 MiB L2) cycled per launch",
                "seed": 1002}

    def bound_of(self, m):
        # ridge of the measured peaks: tensor-bound once flops/bytes exceeds peak_flops/peak_bw
        return "tensor" if m >= 512 else "hbm"


class QdqInt8(Workload):
    """Config 1: x f32 [4096,4096] ~ N(0,1), scale = max|x|/127; one pass writes q (int8) and
    y = q*scale (f32)."""

    name = "config1_int8_qdq_round_trip"
    metric = "Q/DQ HBM GB/s (config 1: per-tensor int8 quantize + dequantize round trip, f32 [4096,4096])"
    unit = "GB/s"
    dtype = "f32 -> int8 -> f32"
    SHAPE = (4096, 4096)
    REPLICAS = 4  # 4 x (64 + 16 + 64) MiB

    def __init__(self, torch, ql, device, seed=1001):
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
        return [("fused_qdq", self.run_part, 0, 9 * n)]

    def e2e_step(self):
        i = self.turn % self.REPLICAS
        self.x[i].copy_(self.x_host, non_blocking=True)
        self.run_part()
        self.q_host.copy_(self.q[i], non_blocking=True)
        self.y_host.copy_(self.y[i], non_blocking=True)

    def e2e_bytes(self):
        n = self.SHAPE[0] * self.SHAPE[1]
        return 4 * n, 5 * n

    def config(self):
        return {"workload": self.name, "shape": list(self.SHAPE), "scale": "max|x|/127 (f32, computed on the GPU)",
                "l2": f"{self.REPLICAS} input/output replicas (576 MiB > 126 MiB L2) cycled per step", "seed": 1001}

    def bound_of(self, _):
        return "hbm"


WORKLOADS = {"c2": W8A16Linear, "c1": QdqInt8}


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
    raise SystemExit(f"no CPU restatement for workload {workload}")


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
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
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": wl.dtype, "data": "synthetic (seeded)",
            "config": {"workload": wl.name, "arm": "CPU restatement of the reference's host path (oracle/ql_oracle.c); "
                       "the reference itself cannot be built here"},
            "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
# the product arm
# ----------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
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
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    wl = WORKLOADS[args.workload](torch, ql, device)
    parts = wl.parts()
    stream = torch.cuda.current_stream(device)
    L = ql.lib()

    # -------- device-resident timing: K steps, every part bracketed by events on the launch stream
    for _ in range(args.warmup):
        for _, fn, _, _ in parts:
            fn()
    barrier()
    clocks = ClockSampler(local)
    clocks.start()
    ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in parts] for _ in range(args.steps)]
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = L.ql_launch_count()
    t_start.record(stream)
    for s in range(args.steps):
        for p, (_, fn, _, _) in enumerate(parts):
            ev[s][p][0].record(stream)
            fn()
            ev[s][p][1].record(stream)
    t_end.record(stream)
    barrier()
    launches = L.ql_launch_count() - launches0
    total_ms = t_start.elapsed_time(t_end)
    clock_info = clocks.stop()
    part_ms = [sum(ev[s][p][0].elapsed_time(ev[s][p][1]) for s in range(args.steps)) / args.steps for p in range(len(parts))]

    # -------- end to end: inputs from pinned host memory, results read back, every step
    for _ in range(3):
        wl.e2e_step()
    barrier()
    e_start, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_start.record(stream)
    for _ in range(args.steps):
        wl.e2e_step()
    e_end.record(stream)
    barrier()
    e2e_ms = e_start.elapsed_time(e_end)

    if dist is not None:
        t = torch.tensor([total_ms, e2e_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, e2e_ms = float(t[0]), float(t[1])

    step_flops = sum(f for _, _, f, _ in parts)
    step_bytes = sum(b for _, _, _, b in parts)
    work = step_flops if wl.unit == "TFLOP/s" else step_bytes
    denom = 1e12 if wl.unit == "TFLOP/s" else 1e9
    value = work * args.steps * world / (total_ms * 1e-3) / denom
    e2e_value = work * args.steps * world / (e2e_ms * 1e-3) / denom

    peaks = measured_peaks()
    dom = max(range(len(parts)), key=lambda p: part_ms[p])
    name, _, f, b = parts[dom]
    m_dom = wl.MS[dom] if hasattr(wl, "MS") else None
    bound = wl.bound_of(m_dom)
    if bound == "tensor":
        achieved, peak, unit = f / (part_ms[dom] * 1e-3) / 1e12, peaks["bf16_tflops_sustained"], "TFLOP/s"
    else:
        achieved, peak, unit = b / (part_ms[dom] * 1e-3) / 1e9, peaks["hbm_gbs"], "GB/s"
    roofline = {"kernel": f"{wl.name}:{name}", "bound": bound, "achieved": achieved, "peak": peak, "unit": unit,
                "frac": achieved / peak, "peak_source": peaks["source"], "traffic": None,
                "algorithmic_bytes_per_launch": b, "algorithmic_flops_per_launch": f, "avg_launch_ms": part_ms[dom]}
    per_part = {}
    for p, (nm, _, f, b) in enumerate(parts):
        per_part[nm] = {"ms": part_ms[p], "GB/s": b / (part_ms[p] * 1e-3) / 1e9, "TFLOP/s": f / (part_ms[p] * 1e-3) / 1e12,
                        "frac_hbm": b / (part_ms[p] * 1e-3) / 1e9 / peaks["hbm_gbs"]}

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    h2d, d2h = wl.e2e_bytes()
    line = {"metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": wl.dtype, "data": "synthetic (seeded)", "config": dict(wl.config(), parallelism="replicas only" if world > 1 else "1 GPU"),
            "clocks": clock_info, "gpu_launches": int(launches),
            "e2e": {"value": e2e_value, "unit": wl.unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / args.steps},
            "roofline": roofline, "parts": per_part}
    if not args.no_cpu_baseline and world == 1:
        v, u, cores, sample = cpu_reference(args.workload)
        line["cpu_baseline"] = {"value": v, "unit": u, "cores": cores, "kind": "port", "sample": sample}
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
