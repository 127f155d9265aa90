"""Quantized Llama-style MLP block (benchmark config 5), tensor-parallel over the GPUs of one box.

    x -> RMSNorm (eps, weight 1) + per-token e4m3 quantize
      -> gate/up projection (fp8 GEMM, per-token x per-output-channel scales in the epilogue)
      -> SwiGLU + per-token e4m3 re-quantize
      -> down projection (fp8 GEMM)  -> sum over ranks (added into every rank's output by the GEMM's
         epilogue through NVSwitch replication, or an NCCL all-reduce where that is unavailable)

Sharding follows the usual column-/row-parallel split: every rank holds `inter / world` columns of
the gate and up projections (no exchange needed before SwiGLU) and the matching rows of the down
projection, whose partial results are summed.  The per-token scale of the re-quantized activation
is local to each rank's columns and is folded into that rank's down-projection epilogue, so no
extra collective is needed.  The reference has no such block operator; its pieces are
tensorrt.quantize / dequantize / matrix_multiply (see include/qlinear_b200.h) composed as
tripy/nvtripy/frontend/module/linear.py:127-151 composes them."""
from __future__ import annotations

import torch

from . import _lib
from . import dtypes as dt
from . import ops
from . import peer
from .linear import gemm_fp8
from .tensor import current_stream, ql_view


def shard_range(n: int, world: int, rank: int):
    """[begin, end) of the slice of `n` columns rank `rank` of `world` owns (n % world == 0)."""
    if n % world:
        raise ValueError(f"{n} columns do not split evenly over {world} ranks")
    per = n // world
    return rank * per, (rank + 1) * per


def quantize_per_channel_fp8(w: torch.Tensor):
    """e4m3 weights with one f32 scale per output channel (row): scale = max|row| / 448."""
    s = ops.amax_scale(w, dt.float8, dim=0, scale_dtype=dt.float32)
    q = torch.empty(w.shape, dtype=torch.float8_e4m3fn, device=w.device)
    ops.quantize_to(w, s, q, dim=0)
    return q, s


def rmsnorm_quant_fp8(x: torch.Tensor, eps: float, q=None, scale=None):
    T, H = x.shape
    q = q if q is not None else torch.empty((T, H), dtype=torch.float8_e4m3fn, device=x.device)
    scale = scale if scale is not None else torch.empty((T,), dtype=torch.float32, device=x.device)
    tx, tq, ts = ql_view(x), ql_view(q), ql_view(scale)
    _lib.check(_lib.lib().ql_rmsnorm_quant_fp8(tx, float(eps), tq, ts, current_stream(x.device)))
    return q, scale


def swiglu_quant_fp8(gate_up: torch.Tensor, q=None, scale=None):
    T, I2 = gate_up.shape
    q = q if q is not None else torch.empty((T, I2 // 2), dtype=torch.float8_e4m3fn, device=gate_up.device)
    scale = scale if scale is not None else torch.empty((T,), dtype=torch.float32, device=gate_up.device)
    tg, tq, ts = ql_view(gate_up), ql_view(q), ql_view(scale)
    _lib.check(_lib.lib().ql_swiglu_quant_fp8(tg, tq, ts, current_stream(gate_up.device)))
    return q, scale


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """[2I, H]: rows of the gate and up projections interleaved in groups of 32 (rows [64b, 64b+32) = gate channels
    [32b, 32b+32), rows [64b+32, 64b+64) = the up channels of the same indices), the layout ql_gemm_fp8_swiglu takes."""
    I, H = w_gate.shape
    return torch.stack([w_gate.reshape(I // 32, 32, H), w_up.reshape(I // 32, 32, H)], dim=1).reshape(2 * I, H).contiguous()


def gemm_fp8_swiglu(xq, wq_gu, sx, s_gu, act, row_amax):
    """act = silu(gate) * up of the gate/up projection (interleaved weights), formed in the GEMM's epilogue;
    row_amax[t] = max|act[t, :]|."""
    _lib.check(_lib.lib().ql_gemm_fp8_swiglu(ql_view(xq), ql_view(wq_gu), ql_view(sx), ql_view(s_gu), ql_view(act), ql_view(row_amax),
                                             current_stream(xq.device)))
    return act, row_amax


def quantize_rows_fp8(act, row_amax, q=None, scale=None):
    """Per-token e4m3 quantize with scale = row_amax / 448: (q, scale)."""
    T, I = act.shape
    q = q if q is not None else torch.empty((T, I), dtype=torch.float8_e4m3fn, device=act.device)
    scale = scale if scale is not None else torch.empty((T,), dtype=torch.float32, device=act.device)
    _lib.check(_lib.lib().ql_quantize_rows_fp8(ql_view(act), ql_view(row_amax), ql_view(q), ql_view(scale), current_stream(act.device)))
    return q, scale


class QuantizedMLP:
    """One rank's shard of the block.  `w_gate`, `w_up`: [inter_local, hidden]; `w_down`: [hidden, inter_local]
    (bf16 / f16, Linear's [out, in] layout).  Weights are quantized once, here."""

    def __init__(self, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, eps: float = 1e-5, group=None,
                 fused_all_reduce="auto", fused_swiglu="auto"):
        """`fused_all_reduce`: True = the down projection's epilogue does the reduction over peer memory
        (qlinear.peer): with two ranks the epilogue adds its partial result into both outputs; with more it adds
        each row into the output of the rank that owns the row, and the owners broadcast.  False = NCCL all-reduce after the GEMM;
        "auto" = over peer memory when the box supports it and the group has several ranks; "scatter" / "switch" /
        "pipeline" = a given protocol whatever the group size (see _buffers).

        The result is an internal buffer (with a peer protocol this rank's replica of one of a few buffers used in
        turn; otherwise one of two local buffers): it stays intact during the next call and is cleared or
        overwritten by the call after that.  Copy it if it must live longer."""
        self.eps, self.group = eps, group
        self._force = fused_all_reduce if fused_all_reduce in ("scatter", "switch", "pipeline") else None   # a protocol on any group size
        self.slabs = 4        # token slabs of the pipelined protocol
        self._comm = None     # side stream of the pipelined protocol
        if fused_all_reduce == "auto":
            fused_all_reduce = group is not None and peer.available(group)
        self.fused_all_reduce = bool(fused_all_reduce) and group is not None
        self._step = 0
        self.hidden, self.inter_local = w_gate.shape[1], w_gate.shape[0]
        self.out_dtype = dt.from_torch(w_gate.dtype)
        # SwiGLU in the gate/up projection's epilogue (the [T, 2I] projection is never written) wherever the shapes
        # allow it: weight rows interleaved in groups of 32, K a multiple of 16 bytes.  Otherwise the projection is
        # written out, rounded to the activation type, and a row kernel applies SwiGLU and quantizes.
        can_fuse = self.inter_local % 32 == 0 and self.hidden % 16 == 0
        self.fused_swiglu = can_fuse if fused_swiglu == "auto" else (bool(fused_swiglu) and can_fuse)
        if self.fused_swiglu:
            self.wq_gu, self.s_gu = quantize_per_channel_fp8(interleave_gate_up(w_gate, w_up))
        else:
            self.wq_gu, self.s_gu = quantize_per_channel_fp8(torch.cat([w_gate, w_up], dim=0).contiguous())
        self.wq_d, self.s_d = quantize_per_channel_fp8(w_down.contiguous())
        self._buf = {}

    def _buffers(self, T, device):
        if self._buf.get("T") != T:
            H, I = self.hidden, self.inter_local
            od = self.out_dtype.torch
            self._buf = {"T": T,
                         "xq": torch.empty((T, H), dtype=torch.float8_e4m3fn, device=device), "sx": torch.empty((T,), dtype=torch.float32, device=device),
                         "gu": None if self.fused_swiglu else torch.empty((T, 2 * I), dtype=od, device=device),
                         "act": torch.empty((T, I), dtype=od, device=device) if self.fused_swiglu else None,
                         "amax": torch.empty((T,), dtype=torch.float32, device=device) if self.fused_swiglu else None,
                         "aq": torch.empty((T, I), dtype=torch.float8_e4m3fn, device=device), "sa": torch.empty((T,), dtype=torch.float32, device=device),
                         # two results used in turn (like the peer protocols' buffers): a caller may still be reading the
                         # previous result, e.g. copying it to the host, while the next call runs
                         "y2": [torch.empty((T, H), dtype=od, device=device) for _ in range(2)]}
            self._buf["y"] = self._buf["y2"][0]
            world = 1
            if self.fused_all_reduce:
                import torch.distributed as dist
                world = dist.get_world_size(self.group)
            # Adding into every output is only used with two ranks: with more, the partial sums would reach each
            # output in a different order and the ranks' results would differ in the last bit (and every GPU would
            # receive world x the data).  Beyond two ranks rows have owners: the epilogue adds each row into its
            # owner's output (the reduce-scatter hides under the GEMM) and the owners broadcast their rows.
            # "switch_reduce" (GEMM into the local replica, then the NVSwitch sums each rank's own rows in f32 and
            # writes them to everyone) rounds every sum once; on two GPUs it was the slowest of the three
            # (1.37 ms per step against 1.23 add_all and 1.31 add_owner), so it serves where rows do not split
            # into owner blocks of 128, or on request.
            owner_ok, switch_ok = world >= 2 and T % (128 * world) == 0, world >= 2 and T % world == 0
            # "switch_pipelined": the down projection runs slab by slab over the tokens into the local replica; as soon
            # as a slab's partial results are out, a side stream does that slab's barrier and in-switch reduction
            # while the main stream computes the next slab, so only the last slab's exchange is exposed.
            slabs = self.slabs
            while slabs > 1 and T % (slabs * world * 8) != 0:
                slabs //= 2
            pipe_ok = switch_ok and slabs > 1
            self._buf["slabs"] = slabs
            if self._force == "pipeline" and pipe_ok:
                self._buf["protocol"] = "switch_pipelined"
            elif self._force == "scatter" and owner_ok:
                self._buf["protocol"] = "add_owner"
            elif self._force == "switch" and switch_ok:
                self._buf["protocol"] = "switch_reduce"
            elif world == 2:
                self._buf["protocol"] = "add_all"
            elif owner_ok:
                self._buf["protocol"] = "add_owner"
            elif switch_ok:
                self._buf["protocol"] = "switch_reduce"
            else:
                self._buf["protocol"] = "nccl"
            if self._buf["protocol"] != "nccl":
                # two output buffers, used in turn: while the ranks add into one, the other is cleared for
                # the next call, and a barrier separates "all added" from "anyone reads"
                # The add protocols clear the buffer of the call after next while they run, so they rotate over three
                # buffers and the one holding the previous result is left alone; the switch protocols need no
                # clearing and rotate over two.  Either way a result stays intact during the next call.
                n_out = 3 if self._buf["protocol"] in ("add_all", "add_owner") else 2
                self._buf["y_peer"] = [peer.PeerTensor((T, H), od, self.group) for _ in range(n_out)]
        return self._buf

    def protocol(self, T, device) -> str:
        """How the down projection's partial sums are combined for `T` tokens: add_all, add_owner, switch_reduce or nccl."""
        return self._buffers(T, device)["protocol"]

    # the four local stages, separately callable so that a benchmark can time them
    def stage_norm_quant(self, x, b):
        rmsnorm_quant_fp8(x, self.eps, b["xq"], b["sx"])

    def stage_gate_up(self, b):
        if self.fused_swiglu:
            gemm_fp8_swiglu(b["xq"], self.wq_gu, b["sx"], self.s_gu, b["act"], b["amax"])
        else:
            gemm_fp8(b["xq"], self.wq_gu, b["sx"], self.s_gu, out_dtype=self.out_dtype, out=b["gu"])

    def stage_swiglu_quant(self, b):
        if self.fused_swiglu:
            quantize_rows_fp8(b["act"], b["amax"], b["aq"], b["sa"])
        else:
            swiglu_quant_fp8(b["gu"], b["aq"], b["sa"])

    def stage_down(self, b):
        gemm_fp8(b["aq"], self.wq_d, b["sa"], self.s_d, out_dtype=self.out_dtype, out=b["y"])

    def stage_all_reduce(self, b):
        if self.group is not None:
            import torch.distributed as dist
            dist.all_reduce(b["y"], group=self.group)

    # the fused form of the last two stages
    def _scatter(self, b):
        """True when rows have owners (reduce-scatter + broadcast); False when every rank adds into every output."""
        return b["protocol"] == "add_owner"

    def _out(self, b):
        """The output buffer of the current call."""
        return b["y_peer"][self._step % len(b["y_peer"])]

    def stage_down_add(self, b):
        mode = peer.ADD_OWNER if self._scatter(b) else peer.ADD_ALL
        peer.gemm_fp8_peer(b["aq"], self.wq_d, b["sa"], self.s_d, self._out(b), mode)

    def stage_clear_next(self, b):
        nxt = b["y_peer"][(self._step + 1) % len(b["y_peer"])]
        if self._scatter(b):   # only the rows this rank owns are added into; the rest is overwritten by broadcasts
            rows = b["T"] // nxt.world
            nxt.local[nxt.rank * rows:(nxt.rank + 1) * rows].zero_()
        else:
            nxt.local.zero_()

    def stage_barrier(self, b):
        self._out(b).barrier()

    def stage_broadcast_owned(self, b):
        y = self._out(b)
        rows = b["T"] // y.world
        y.broadcast_rows(y.rank * rows, rows)

    # the switch protocol: plain GEMM into the local replica, then the in-switch sum of the owned rows
    def stage_down_local(self, b):
        gemm_fp8(b["aq"], self.wq_d, b["sa"], self.s_d, out_dtype=self.out_dtype, out=self._out(b).local)

    def stage_switch_reduce_owned(self, b):
        y = self._out(b)
        rows = b["T"] // y.world
        y.reduce_rows(y.rank * rows, rows)

    # the pipelined switch protocol: one slab of tokens at a time
    def stage_down_slab(self, b, s):
        rows = b["T"] // b["slabs"]
        sl = slice(s * rows, (s + 1) * rows)
        gemm_fp8(b["aq"][sl], self.wq_d, b["sa"][sl], self.s_d, out_dtype=self.out_dtype, out=self._out(b).local[sl])

    def stage_reduce_slab(self, b, s):
        """Barrier (every rank's partial results of slab `s` are in its replica), then the in-switch sum of the
        rows of the slab this rank owns, written to every replica.  Runs on the current stream."""
        y = self._out(b)
        rows = b["T"] // b["slabs"]
        mine = rows // y.world
        y.barrier()
        y.reduce_rows(s * rows + y.rank * mine, mine)

    def comm_stream(self, device):
        if self._comm is None:
            self._comm = torch.cuda.Stream(device, priority=-1)
        return self._comm

    def _forward_pipelined(self, b, device):
        main, comm = torch.cuda.current_stream(device), self.comm_stream(device)
        for s in range(b["slabs"]):
            self.stage_down_slab(b, s)
            done = main.record_event()
            with torch.cuda.stream(comm):
                comm.wait_event(done)
                self.stage_reduce_slab(b, s)
        main.wait_stream(comm)
        self.stage_barrier(b)               # every rank's rows of every slab have been written everywhere
        y = self._out(b).local
        self._step += 1
        return y

    def reset_peer_buffers(self):
        """Zero every output buffer on every rank (after anything that added into them out of turn)."""
        for t in self._buf.get("y_peer", []):
            t.barrier()
            t.local.zero_()
            t.barrier()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        b = self._buffers(x.shape[0], x.device)
        self.stage_norm_quant(x, b)
        self.stage_gate_up(b)
        self.stage_swiglu_quant(b)
        if b["protocol"] == "switch_pipelined":
            return self._forward_pipelined(b, x.device)
        if b["protocol"] == "switch_reduce":
            self.stage_down_local(b)
            self.stage_barrier(b)           # every rank's partial result is in its own replica
            self.stage_switch_reduce_owned(b)
            self.stage_barrier(b)           # every rank's rows have been summed and written everywhere
            y = self._out(b).local
            self._step += 1
            return y
        if b["protocol"] != "nccl":
            self.stage_down_add(b)
            self.stage_clear_next(b)
            self.stage_barrier(b)           # every rank's partial sums have landed
            if self._scatter(b):
                self.stage_broadcast_owned(b)
                self.stage_barrier(b)       # every rank's rows have landed
            y = self._out(b).local
            self._step += 1
            return y
        b["y"] = b["y2"][self._step % 2]
        self._step += 1
        self.stage_down(b)
        self.stage_all_reduce(b)
        return b["y"]

    __call__ = forward
