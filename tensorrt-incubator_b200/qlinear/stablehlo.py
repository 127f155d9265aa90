"""A front door for compiled programs: reads the StableHLO text of a function on the quantized-linear
path and runs it on the library's kernels.

The reference recognises quantize / dequantize in three spellings and this module accepts the same three:

* the arithmetic decomposition  divide -> round_nearest_even -> clamp -> convert  (quantize) and
  convert -> multiply  (dequantize) with the scale reaching the data through `broadcast_in_dim`
  (dims = [] per tensor, dims = [axis] per channel, dims = [1, 2] + `reshape` for blocks), exactly the
  shapes `stablehlo-raise-qdq` matches
  (mlir-tensorrt/compiler/lib/Dialect/StablehloExt/Transforms/StablehloRaiseQDQ.cpp:138-265, 348-418);
* `stablehlo.composite "tensorrt.pt_q|pc_q|block_q|pt_dq|pc_dq|block_dq"` with `composite_attributes =
  {axis, scale}` (what that pass produces, StablehloRaiseQDQ.cpp:270-345);
* `stablehlo.custom_call @tensorrt.quantize / @tensorrt.dequantize` with `mode` and `axis` attributes, and
  `@tensorrt.dynamic_quantize` (two results: NVFP4 data and block scales)
  (what the JAX plug-in emits, integrations/PJRT/python/mlir_tensorrt_jax/mtrt_ops/quantize.py:134; examples
  in compiler/test/Passes/0_Frontend/StablehloToTensorRT/stablehlo-to-tensorrt-trt10.mlir:401-440).

A float8 quantize written as the decomposition rounds to an integer before the conversion (that is what the
arithmetic says); the composite and custom_call spellings mean TensorRT's operator, which converts directly.

`stablehlo.dot_general` over a (transposed) dequantized int8 / int4 weight becomes the weight-only
linear kernel; other 16-bit contractions use the tensor-core GEMM.  Anything else is refused: this is not
a StableHLO interpreter, only the hot path's matcher.  Parsing needs no GPU; running does."""
from __future__ import annotations

import re
from dataclasses import dataclass, field

import numpy as np
import torch

from . import _lib
from . import dtypes as dt
from .linear import linear as _linear_nt, linear_w4a16 as _linear_w4a16, linear_w8a16 as _linear_w8a16
from . import ops
from .tensor import Float4Tensor, Int4Tensor, current_stream, empty_quantized, ql_view

_ELEM = {"f32": dt.float32, "f16": dt.float16, "bf16": dt.bfloat16, "i8": dt.int8, "i4": dt.int4, "f8E4M3FN": dt.float8,
         "f4E2M1FN": dt.float4}
_BOUNDS = {dt.int8: (-128.0, 127.0), dt.int4: (-8.0, 7.0), dt.float8: (-448.0, 448.0)}


class UnsupportedProgram(ValueError):
    """The function contains something outside the quantized-linear path."""


@dataclass
class TensorType:
    shape: tuple
    elem: str

    @staticmethod
    def parse(text: str) -> "TensorType":
        m = re.fullmatch(r"tensor<(.*)>", text.strip())
        if not m:
            raise UnsupportedProgram(f"not a ranked tensor type: {text}")
        parts = m.group(1).split("x")
        elem = parts[-1]
        dims = parts[:-1]
        if any(not d.isdigit() for d in dims):
            raise UnsupportedProgram(f"dynamic shapes are not supported: {text}")
        if elem not in _ELEM:
            raise UnsupportedProgram(f"element type {elem} is not on the quantized-linear path")
        return TensorType(tuple(int(d) for d in dims), elem)

    @property
    def dtype(self) -> dt.dtype:
        return _ELEM[self.elem]


# symbolic values while matching ---------------------------------------------------------------
@dataclass
class Val:
    kind: str                 # arg | const | bcast | div | round | clamp | real
    type: TensorType
    src: tuple = ()           # operand Vals
    data: np.ndarray | None = None   # constants
    attrs: dict = field(default_factory=dict)
    slot: int | None = None   # runtime slot for arg / real values


@dataclass
class Step:
    op: str                   # quantize | dequantize | linear_w8a16 | linear_w4a16 | matmul16
    out: int
    ins: tuple
    attrs: dict


def _parse_dense(text: str, ty: TensorType) -> np.ndarray:
    body = text.strip()
    if body.startswith("dense_resource") or "__elided__" in body:
        raise UnsupportedProgram("elided constants cannot be executed")
    m = re.fullmatch(r"dense<(.*)>", body, flags=re.S)
    if not m:
        raise UnsupportedProgram(f"unsupported constant: {text[:60]}")
    inner = m.group(1).replace("[", " ").replace("]", " ").replace(",", " ")
    vals = np.array([float(v) for v in inner.split()], dtype=np.float64)
    n = int(np.prod(ty.shape)) if ty.shape else 1
    if vals.size == 1:
        vals = np.full(n, vals[0])
    if vals.size != n:
        raise UnsupportedProgram("constant does not match its type")
    return vals.reshape(ty.shape)


def _split_top(text: str, sep: str = ",") -> list[str]:
    out, depth, cur = [], 0, ""
    for ch in text:
        if ch in "<[({":
            depth += 1
        elif ch in ">])}":
            depth -= 1
        if ch == sep and depth == 0:
            out.append(cur.strip())
            cur = ""
        else:
            cur += ch
    if cur.strip():
        out.append(cur.strip())
    return out


class Program:
    """A matched function: `steps` over numbered slots, runnable on CUDA torch tensors."""

    def __init__(self, name, arg_types, result_slots, result_types, steps, constants):
        self.name, self.arg_types, self.result_slots, self.result_types = name, arg_types, result_slots, result_types
        self.steps, self.constants = steps, constants

    # ------------------------------------------------------------------------------------------
    @staticmethod
    def from_text(text: str, func: str | None = None) -> "Program":
        text = "\n".join(l for l in text.splitlines() if not l.strip().startswith("//"))
        m = None
        for cand in re.finditer(r"func\.func\s+(?:public\s+|private\s+)?@([\w.$-]+)\s*\((.*?)\)\s*->\s*(.*?)\s*(?:attributes\s*\{.*?\}\s*)?\{", text, flags=re.S):
            if func is None or cand.group(1) == func:
                m = cand
                break
        if m is None:
            raise UnsupportedProgram(f"function {func or '(first)'} not found")
        name = m.group(1)
        body_start = m.end()
        depth, i = 1, body_start
        while depth and i < len(text):
            depth += {"{": 1, "}": -1}.get(text[i], 0)
            i += 1
        body = text[body_start:i - 1]

        vals: dict[str, Val] = {}
        arg_types, n_slots = [], 0
        for a in _split_top(m.group(2)):
            am = re.fullmatch(r"(%[\w.#-]+)\s*:\s*(tensor<[^>]*>).*", a, flags=re.S)
            if not am:
                raise UnsupportedProgram(f"unsupported argument: {a}")
            ty = TensorType.parse(am.group(2))
            vals[am.group(1)] = Val("arg", ty, slot=n_slots)
            arg_types.append(ty)
            n_slots += 1

        steps: list[Step] = []
        constants: dict[int, tuple] = {}
        result_slots, result_types = [], []

        def new_slot():
            nonlocal n_slots
            n_slots += 1
            return n_slots - 1

        def realise(v: Val) -> int:
            """Slot holding v at run time (arguments, results of steps, materialised constants)."""
            if v.slot is not None:
                return v.slot
            if v.kind == "const":
                v.slot = new_slot()
                constants[v.slot] = (v.data, v.type)
                return v.slot
            raise UnsupportedProgram(f"a {v.kind} value is used outside a quantize/dequantize pattern")

        def scale_of(b: Val):
            """(scale Val, mode, axis) from the broadcast that feeds divide / multiply."""
            if b.kind == "const" and b.type.shape == ():
                return b, "pt", None
            if b.kind == "reshape" and b.src[0].kind == "bcast" and b.src[0].attrs["dims"] == [1, 2]:
                return b.src[0].src[0], "block", None
            # the reference insists on a constant scale; the kernels read it from device memory, so a
            # function argument serves as well
            if b.kind != "bcast" or b.src[0].kind not in ("const", "arg"):
                raise UnsupportedProgram("the scale must be a constant or an argument reaching the data through broadcast_in_dim")
            dims = b.attrs["dims"]
            if dims == []:
                return b.src[0], "pt", None
            if len(dims) == 1:
                return b.src[0], "pc", dims[0]
            raise UnsupportedProgram(f"unsupported scale broadcast dims {dims}")

        def emit_q(x: Val, scale_v: Val, mode: str, axis, out_ty: TensorType, fp8_mode: str) -> Val:
            s_slot = realise(scale_v)
            out = Val("real", out_ty, slot=new_slot())
            steps.append(Step("quantize", out.slot, (realise(x), s_slot),
                              {"dtype": out_ty.dtype, "mode": mode, "axis": axis, "fp8_mode": fp8_mode}))
            return out

        def emit_dq(q: Val, scale_v: Val, mode: str, axis, out_ty: TensorType) -> Val:
            out = Val("real", out_ty, slot=new_slot())
            out.attrs.update(dq_of=q, dq_scale=scale_v, dq_mode=mode, dq_axis=axis)
            steps.append(Step("dequantize", out.slot, (realise(q), realise(scale_v)), {"dtype": out_ty.dtype, "mode": mode, "axis": axis}))
            return out

        for raw in re.split(r"\n(?=\s*(?:%|return|func\.return|stablehlo\.return))", body):
            line = " ".join(raw.split())
            if not line:
                continue
            if line.startswith(("return", "func.return")):
                rm = re.match(r"(?:func\.)?return\s+(.*?)\s*:\s*(.*)", line)
                for nm, ty in zip(_split_top(rm.group(1)), _split_top(rm.group(2))):
                    result_slots.append(realise(vals[nm]))
                    result_types.append(TensorType.parse(ty))
                continue
            dq = re.match(r"(%[\w.-]+):2\s*=\s*stablehlo\.custom_call\s+@tensorrt\.dynamic_quantize\((%[\w.#-]+),\s*(%[\w.#-]+)\)\s*\{(.*)\}\s*:"
                          r"\s*\(.*\)\s*->\s*\((.*)\)$", line)
            if dq:
                # NVFP4: two results, %name#0 (e2m1 data) and %name#1 (e4m3 block scales)
                name2, x, gs, attrs = dq.group(1), vals[dq.group(2)], vals[dq.group(3)], dq.group(4)
                tys = [TensorType.parse(t) for t in _split_top(dq.group(5))]
                axis = int(re.search(r"axis\s*=\s*(-?\d+)", attrs).group(1))
                bm = re.search(r"block_size\s*=\s*(\d+)", attrs)
                data, scales = Val("real", tys[0], slot=new_slot()), Val("real", tys[1], slot=new_slot())
                steps.append(Step("dynamic_quantize", data.slot, (realise(x), realise(gs)),
                                  {"axis": axis, "block_size": int(bm.group(1)) if bm else 16, "scales_slot": scales.slot}))
                vals[name2 + "#0"], vals[name2 + "#1"] = data, scales
                continue
            lm = re.match(r"(%[\w.#-]+)\s*=\s*(.*)", line)
            if not lm:
                raise UnsupportedProgram(f"cannot read: {line[:80]}")
            res, rhs = lm.group(1), lm.group(2)
            types = rhs.rsplit(" : ", 1)[1] if " : " in rhs else ""
            out_ty = TensorType.parse(types.split("->")[-1].strip()) if types else None

            if rhs.startswith("stablehlo.constant"):
                cm = re.match(r"stablehlo\.constant\s+(.*)\s:\s*(tensor<[^>]*>)$", rhs, flags=re.S)
                ty = TensorType.parse(cm.group(2))
                vals[res] = Val("const", ty, data=_parse_dense(cm.group(1), ty))
            elif rhs.startswith("stablehlo.broadcast_in_dim"):
                bm = re.match(r"stablehlo\.broadcast_in_dim\s+(%[\w.#-]+),\s*dims\s*=\s*\[([\d,\s]*)\]", rhs)
                dims = [int(d) for d in bm.group(2).replace(" ", "").split(",") if d]
                vals[res] = Val("bcast", out_ty, (vals[bm.group(1)],), attrs={"dims": dims})
            elif rhs.startswith("stablehlo.reshape"):
                src = vals[re.match(r"stablehlo\.reshape\s+(%[\w.#-]+)", rhs).group(1)]
                vals[res] = Val("reshape", out_ty, (src,))
            elif rhs.startswith("stablehlo.divide"):
                a, b = re.match(r"stablehlo\.divide\s+(%[\w.#-]+),\s*(%[\w.#-]+)", rhs).groups()
                vals[res] = Val("div", out_ty, (vals[a], vals[b]))
            elif rhs.startswith("stablehlo.round_nearest_even"):
                a = re.match(r"stablehlo\.round_nearest_even\s+(%[\w.#-]+)", rhs).group(1)
                vals[res] = Val("round", out_ty, (vals[a],))
            elif rhs.startswith("stablehlo.clamp"):
                lo, a, hi = re.match(r"stablehlo\.clamp\s+(%[\w.#-]+),\s*(%[\w.#-]+),\s*(%[\w.#-]+)", rhs).groups()
                vals[res] = Val("clamp", out_ty, (vals[lo], vals[a], vals[hi]))
            elif rhs.startswith("stablehlo.convert"):
                a = vals[re.match(r"stablehlo\.convert\s+(%[\w.#-]+)", rhs).group(1)]
                if out_ty.dtype in dt.QUANTIZED_DTYPES:
                    # tail of the quantize decomposition
                    if a.kind != "clamp" or a.src[1].kind != "round" or a.src[1].src[0].kind != "div":
                        raise UnsupportedProgram("convert to a quantized type must end divide -> round_nearest_even -> clamp")
                    lo, hi = a.src[0], a.src[2]
                    want = _BOUNDS[out_ty.dtype]
                    if lo.kind != "const" or hi.kind != "const" or (float(lo.data.reshape(-1)[0]), float(hi.data.reshape(-1)[0])) != want:
                        raise UnsupportedProgram(f"clamp bounds do not match {out_ty.elem}")
                    div = a.src[1].src[0]
                    scale_v, mode, axis = scale_of(div.src[1])
                    vals[res] = emit_q(div.src[0], scale_v, mode, axis, out_ty, "stablehlo")
                elif a.type.dtype in dt.QUANTIZED_DTYPES:
                    vals[res] = Val("widened", out_ty, (a,))  # head of the dequantize decomposition
                elif a.kind == "const":
                    # clamp bounds of 16-bit programs are f32 constants converted to the data type
                    vals[res] = Val("const", out_ty, data=a.data)
                else:
                    raise UnsupportedProgram("only conversions to or from quantized types are on this path")
            elif rhs.startswith("stablehlo.multiply"):
                a, b = (vals[n] for n in re.match(r"stablehlo\.multiply\s+(%[\w.#-]+),\s*(%[\w.#-]+)", rhs).groups())
                if b.kind == "widened":
                    a, b = b, a
                if a.kind != "widened":
                    raise UnsupportedProgram("multiply is only supported as the tail of a dequantize")
                scale_v, mode, axis = scale_of(b)
                vals[res] = emit_dq(a.src[0], scale_v, mode, axis, out_ty)
            elif rhs.startswith("stablehlo.composite"):
                cm = re.match(r'stablehlo\.composite\s+"tensorrt\.(pt|pc|block)_(q|dq)"\s+(%[\w.#-]+)\s*\{(.*)\}\s*:', rhs, flags=re.S)
                if not cm:
                    raise UnsupportedProgram(f"unsupported composite: {rhs[:80]}")
                mode, which, x = cm.group(1), cm.group(2), vals[cm.group(3)]
                attrs = cm.group(4)
                axis_m = re.search(r"axis\s*=\s*(-?\d+)", attrs)
                axis = int(axis_m.group(1)) if axis_m and int(axis_m.group(1)) >= 0 and mode == "pc" else None
                sm = re.search(r"scale\s*=\s*(dense<.*?>)\s*:\s*(tensor<[^>]*>)", attrs, flags=re.S)
                sty = TensorType.parse(sm.group(2))
                scale_v = Val("const", sty, data=_parse_dense(sm.group(1), sty))
                vals[res] = emit_q(x, scale_v, mode, axis, out_ty, "direct") if which == "q" else emit_dq(x, scale_v, mode, axis, out_ty)
            elif rhs.startswith("stablehlo.custom_call"):
                cm = re.match(r"stablehlo\.custom_call\s+@tensorrt\.(quantize|dequantize)\((%[\w.#-]+),\s*(%[\w.#-]+)\)\s*\{(.*)\}\s*:", rhs, flags=re.S)
                if not cm:
                    raise UnsupportedProgram(f"unsupported custom_call: {rhs[:80]}")
                which, x, s, attrs = cm.group(1), vals[cm.group(2)], vals[cm.group(3)], cm.group(4)
                mode = re.search(r'mode\s*=\s*"tensorrt\.(pt|pc|block)_d?q"', attrs).group(1)
                axis_m = re.search(r"axis\s*=\s*(-?\d+)", attrs)
                axis = int(axis_m.group(1)) if axis_m and mode == "pc" else None
                vals[res] = emit_q(x, s, mode, axis, out_ty, "direct") if which == "quantize" else emit_dq(x, s, mode, axis, out_ty)
            elif rhs.startswith("stablehlo.transpose"):
                tm = re.match(r"stablehlo\.transpose\s+(%[\w.#-]+),\s*dims\s*=\s*\[([\d,\s]*)\]", rhs)
                if [int(d) for d in tm.group(2).split(",")] != [1, 0]:
                    raise UnsupportedProgram("only 2-D transposes are on this path")
                vals[res] = Val("transposed", out_ty, (vals[tm.group(1)],))
            elif rhs.startswith("stablehlo.dot_general"):
                dm = re.match(r"stablehlo\.dot_general\s+(%[\w.#-]+),\s*(%[\w.#-]+),\s*contracting_dims\s*=\s*\[(\d+)\]\s*x\s*\[(\d+)\]", rhs)
                if not dm:
                    raise UnsupportedProgram("only plain 2-D contractions are on this path")
                a, b, ca, cb = vals[dm.group(1)], vals[dm.group(2)], int(dm.group(3)), int(dm.group(4))
                if len(a.type.shape) != 2 or len(b.type.shape) != 2 or ca != 1:
                    raise UnsupportedProgram("dot_general must contract the last dimension of a 2-D lhs")
                # bring the rhs to [N, K] (Linear's weight layout)
                if b.kind == "transposed" and cb == 0:
                    w = b.src[0]
                elif cb == 1:
                    w = b
                else:
                    raise UnsupportedProgram("the rhs must be [N, K], or [K, N] written as a transpose of [N, K]")
                if out_ty.dtype not in (dt.float16, dt.bfloat16):
                    raise UnsupportedProgram("only 16-bit contractions run on the tensor-core path")
                out = Val("real", out_ty, slot=new_slot())
                q = w.attrs.get("dq_of")
                if q is not None and q.type.dtype is dt.int8 and w.attrs["dq_mode"] == "pc" and w.attrs["dq_axis"] == 0 and q.type.shape[1] % 64 == 0:
                    steps.append(Step("linear_w8a16", out.slot, (realise(a), realise(q), realise(w.attrs["dq_scale"])), {}))
                elif q is not None and q.type.dtype is dt.int4 and w.attrs["dq_mode"] == "block" and w.attrs["dq_scale"].type.shape[0] == q.type.shape[0] \
                        and (q.type.shape[1] // w.attrs["dq_scale"].type.shape[1]) % 128 == 0:
                    steps.append(Step("linear_w4a16", out.slot, (realise(a), realise(q), realise(w.attrs["dq_scale"])), {}))
                else:
                    steps.append(Step("matmul16", out.slot, (realise(a), realise(w)), {}))
                vals[res] = out
            else:
                raise UnsupportedProgram(f"operation outside the quantized-linear path: {rhs.split()[0]}")

        # drop dequantize steps whose only consumer was fused into a weight-only linear
        used = set(result_slots)
        for st in steps:
            used.update(st.ins)
        steps = [st for st in steps if st.op != "dequantize" or st.out in used]
        return Program(name, arg_types, result_slots, result_types, steps, constants)

    # ------------------------------------------------------------------------------------------
    def __call__(self, *args, device="cuda"):
        """Run on CUDA torch tensors (int4 arguments as `Int4Tensor`); returns the function's results."""
        if len(args) != len(self.arg_types):
            raise ValueError(f"{self.name} takes {len(self.arg_types)} arguments")
        slots: dict[int, object] = dict(enumerate(args))
        for slot, (data, ty) in self.constants.items():
            slots[slot] = _materialise(data, ty, device)
        for st in self.steps:
            ins = [slots[i] for i in st.ins]
            if st.op == "quantize":
                x, s = ins
                x = x.contiguous()
                out = empty_quantized(x.shape, st.attrs["dtype"], x.device)
                slots[st.out] = ops.quantize_to(x, s.contiguous(), out, st.attrs["axis"], fp8_mode=st.attrs["fp8_mode"])
            elif st.op == "dynamic_quantize":
                x, gs = ins
                slots[st.out], slots[st.attrs["scales_slot"]] = ops.dynamic_quantize(x, gs, st.attrs["axis"], st.attrs["block_size"])
            elif st.op == "dequantize":
                q, s = ins
                q = q if isinstance(q, (Int4Tensor, Float4Tensor)) else q.contiguous()
                y = torch.empty(tuple(q.shape), dtype=st.attrs["dtype"].torch, device=q.device)
                s = s.contiguous()
                _lib.check(_lib.lib().ql_dequantize(ql_view(q), ql_view(s), ql_view(y), _lib.make_attrs(st.attrs["axis"]),
                                                    current_stream(y.device)))
                slots[st.out] = y
            elif st.op == "linear_w8a16":
                x, q, s = ins
                slots[st.out] = _linear_w8a16(x.contiguous(), q, s.contiguous())
            elif st.op == "linear_w4a16":
                x, q, s = ins
                slots[st.out] = _linear_w4a16(x.contiguous(), q, s.contiguous())
            elif st.op == "matmul16":
                x, w = ins
                slots[st.out] = _linear_nt(x.contiguous(), w.contiguous())
        outs = [slots[i] for i in self.result_slots]
        return outs[0] if len(outs) == 1 else tuple(outs)


def _materialise(data: np.ndarray, ty: TensorType, device):
    """A constant of the program as a device tensor of its declared type."""
    if ty.dtype in dt.QUANTIZABLE_DTYPES:
        return torch.from_numpy(np.array(data, dtype=np.float32).reshape(ty.shape)).to(ty.dtype.torch).to(device)
    ints = torch.from_numpy(np.array(data, dtype=np.int64).reshape(ty.shape)).to(torch.int8)
    if ty.dtype is dt.int8:
        return ints.to(device)
    if ty.dtype is dt.int4:
        return Int4Tensor.pack(ints.to(device))
    raise UnsupportedProgram(f"constants of type {ty.elem} are not supported")
