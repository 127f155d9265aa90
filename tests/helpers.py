"""Conversions between torch tensors (what the product computes on) and the numpy arrays / type
codes the CPU oracle takes, plus seeded input generators shaped like the benchmark configs."""
import numpy as np
import torch

import oracle as orc
import qlinear as ql

CODE_OF_TORCH = {torch.float32: orc.F32, torch.float16: orc.F16, torch.bfloat16: orc.BF16,
                 torch.int8: orc.I8, torch.float8_e4m3fn: orc.F8E4M3}
QL_OF_CODE = {orc.F32: ql.float32, orc.F16: ql.float16, orc.BF16: ql.bfloat16, orc.I8: ql.int8, orc.I4: ql.int4,
              orc.F8E4M3: ql.float8}
TORCH_OF_CODE = {orc.F32: torch.float32, orc.F16: torch.float16, orc.BF16: torch.bfloat16}


def to_np(t):
    """Bit-preserving torch -> numpy: bf16 as uint16, e4m3 as uint8, int4 as packed uint8."""
    if isinstance(t, ql.Int4Tensor):
        return t.packed.cpu().numpy()
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8).numpy()
    return t.numpy()


def code_of(t):
    if isinstance(t, ql.Int4Tensor):
        return orc.I4
    return CODE_OF_TORCH[t.dtype]


def randn(shape, dtype, seed, std=1.0, device="cuda"):
    """N(0, std) drawn on the host in f32 from a seeded generator, rounded to `dtype`."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(shape, generator=g, dtype=torch.float32) * std
    return x.to(dtype).to(device)


def float_values(t):
    """Any float-like torch tensor as float32 numpy values."""
    return t.detach().float().cpu().numpy()


def assert_close_rel(got, want, rel, what=""):
    """|got - want| <= rel * max(|want|, scale) elementwise, scale = rms(want): the tolerance of
    the benchmark's contract for float outputs, guarded against cancellation near zero."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    scale = float(np.sqrt(np.mean(want * want))) if want.size else 0.0
    bound = rel * np.maximum(np.abs(want), scale)
    bad = np.abs(got - want) > bound
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} outside rel {rel}; worst {np.abs(got - want).max()} (rms {scale})"
