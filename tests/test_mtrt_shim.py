"""The executor runtime's CUDA-module boundary (mtrt_cuda_*), the symbols generated host code
calls.  Modelled on the reference's launch-ABI tests
(compiler/test/IntegrationTests/CUDA/cuda-launch-kernel.mlir: a memref plus i32 and f32 scalar
arguments; EmitC/cuda-launch-argpack.mlir:19-21: the missing-artifact error path)."""
import ctypes
import os

import numpy as np
import pytest
import torch

from conftest import ROOT

import oracle as orc
import qlinear as ql
from qlinear import _lib

PTX = os.path.join(ROOT, "tests", "golden", "add_scalar.ptx")


@pytest.fixture(scope="module")
def rt():
    L = ctypes.CDLL(_lib.LIB_PATH)
    vp = ctypes.c_void_p
    L.mtrt_cuda_module_load_from_ptx.argtypes = [ctypes.c_char_p, ctypes.c_size_t]
    L.mtrt_cuda_module_load_from_ptx.restype = vp
    L.mtrt_cuda_module_load_from_ptx_file.argtypes = [ctypes.c_char_p, ctypes.c_size_t]
    L.mtrt_cuda_module_load_from_ptx_file.restype = vp
    L.mtrt_cuda_module_unload.argtypes = [vp]
    L.mtrt_cuda_module_get_function.argtypes = [vp, ctypes.c_char_p, ctypes.c_int64]
    L.mtrt_cuda_module_get_function.restype = vp
    L.mtrt_cuda_launch_kernel.argtypes = [vp] + [ctypes.c_int32] * 7 + [vp, ctypes.POINTER(vp)]
    L.mtrt_cuda_last_error.restype = ctypes.c_char_p
    L.ql_mtrt_bind_kernel.argtypes = [ctypes.c_char_p, ctypes.c_char_p]
    L.mtrt_cuda_stream_create.restype = vp
    L.mtrt_cuda_stream_sync.argtypes = [vp]
    L.mtrt_cuda_stream_destroy.argtypes = [vp]
    L.mtrt_cuda_alloc_async.argtypes = [vp, ctypes.c_int64, ctypes.c_int32, ctypes.c_int8, ctypes.c_int8]
    L.mtrt_cuda_alloc_async.restype = vp
    L.mtrt_cuda_memcpy_async.argtypes = [vp, vp, vp, ctypes.c_int64]
    L.mtrt_cuda_free.argtypes = [vp, vp, ctypes.c_int8, ctypes.c_int8]
    return L


def _args(*values):
    """void** args: each entry points at one kernel parameter."""
    holders = list(values)
    arr = (ctypes.c_void_p * len(holders))(*[ctypes.cast(ctypes.byref(h), ctypes.c_void_p) for h in holders])
    return arr, holders


def test_handles_without_a_gpu(rt):
    ptx = open(PTX, "rb").read()
    mod = rt.mtrt_cuda_module_load_from_ptx(ptx, len(ptx))
    assert mod
    name = b"ql:quantize;in=f32;out=i8;scale=f32;shape=4x4_trailing_bytes_are_ignored"
    fn = rt.mtrt_cuda_module_get_function(mod, name, len(b"ql:quantize;in=f32;out=i8;scale=f32;shape=4x4"))
    assert fn  # the name is length-delimited, not NUL-terminated
    assert rt.ql_mtrt_bind_kernel(b"main_kernel_0", b"ql:dequantize;in=i8;out=f32;scale=f32;shape=8") == 0
    assert rt.mtrt_cuda_module_get_function(mod, b"main_kernel_0", 13)
    assert rt.ql_mtrt_bind_kernel(b"bad", b"not a spec") != 0
    rt.mtrt_cuda_module_unload(mod)
    # missing artifact: an error, not an abort
    missing = b"/nonexistent/kernels.ptx"
    assert not rt.mtrt_cuda_module_load_from_ptx_file(missing, len(missing))
    assert b"could not open artifact" in rt.mtrt_cuda_last_error()


@pytest.mark.gpu
def test_jit_kernel_from_caller_ptx_with_memref_and_scalar_args(rt):
    """A kernel the library does not own goes through the driver JIT exactly as in the reference."""
    mod = rt.mtrt_cuda_module_load_from_ptx_file(PTX.encode(), len(PTX))
    assert mod, rt.mtrt_cuda_last_error()
    fn = rt.mtrt_cuda_module_get_function(mod, b"add_scalar", 10)
    assert fn, rt.mtrt_cuda_last_error()
    stream = rt.mtrt_cuda_stream_create()
    n = 1000
    host = np.arange(n, dtype=np.float32)
    dev = rt.mtrt_cuda_alloc_async(stream, n * 4, 16, 0, 0)
    rt.mtrt_cuda_memcpy_async(stream, host.ctypes.data, dev, n * 4)
    arr, keep = _args(ctypes.c_void_p(dev), ctypes.c_int32(n), ctypes.c_float(2.5))
    rt.mtrt_cuda_launch_kernel(fn, (n + 127) // 128, 1, 1, 128, 1, 1, 0, stream, arr)
    out = np.zeros(n, dtype=np.float32)
    rt.mtrt_cuda_memcpy_async(stream, dev, out.ctypes.data, n * 4)
    rt.mtrt_cuda_stream_sync(stream)
    assert np.array_equal(out, host + np.float32(2.5))
    rt.mtrt_cuda_free(stream, dev, 0, 0)
    rt.mtrt_cuda_stream_sync(stream)
    rt.mtrt_cuda_stream_destroy(stream)
    assert not rt.mtrt_cuda_module_get_function(mod, b"no_such_kernel", 14)
    rt.mtrt_cuda_module_unload(mod)


@pytest.mark.gpu
def test_prebuilt_cubin_artifact_loads_like_ptx(rt, tmp_path):
    """The module data of a compiled program may be a cubin instead of PTX (cuda.compiled_module, kind and data as in
    compiler/include/mlir-tensorrt/Dialect/CUDA/IR/CUDAOps.td:157-215): the same entry points take it."""
    import shutil
    import subprocess
    ptxas = shutil.which("ptxas") or "/usr/local/cuda/bin/ptxas"
    if not os.path.exists(ptxas):
        pytest.skip("no ptxas on this machine to make a cubin from the test artifact")
    cubin = tmp_path / "add_scalar.cubin"
    subprocess.run([ptxas, "-arch=sm_100a", "-o", str(cubin), PTX], check=True)
    path = str(cubin).encode()
    mod = rt.mtrt_cuda_module_load_from_ptx_file(path, len(path))
    assert mod, rt.mtrt_cuda_last_error()
    fn = rt.mtrt_cuda_module_get_function(mod, b"add_scalar", 10)
    assert fn, rt.mtrt_cuda_last_error()
    n = 777
    x = torch.arange(n, dtype=torch.float32, device="cuda")
    arr, keep = _args(ctypes.c_void_p(x.data_ptr()), ctypes.c_int32(n), ctypes.c_float(-1.5))
    rt.mtrt_cuda_launch_kernel(fn, (n + 63) // 64, 1, 1, 64, 1, 1, 0, torch.cuda.current_stream().cuda_stream, arr)
    torch.cuda.synchronize()
    assert torch.equal(x.cpu(), torch.arange(n, dtype=torch.float32) - 1.5)
    rt.mtrt_cuda_module_unload(mod)


def test_manifest_file_maps_compiler_names_to_library_kernels(tmp_path):
    """QL_MTRT_MANIFEST: lines `name = ql:...` bind the names a compiler already emits (read once per process, so the
    check runs in a child process; resolving a library kernel needs no GPU)."""
    import subprocess
    import sys
    manifest = tmp_path / "kernels.manifest"
    manifest.write_text("# kernels of program main\n"
                        "main_quantize_kernel_0 = ql:quantize;in=f32;out=i8;scale=f32;shape=4096x4096\n"
                        "main_linear_kernel_3 = ql:linear_w8a16;x=bf16;scale=f16;M=16;N=11008;K=4096\n")
    code = f"""
import ctypes
L = ctypes.CDLL({_lib.LIB_PATH!r})
L.mtrt_cuda_module_load_from_ptx.argtypes = [ctypes.c_char_p, ctypes.c_size_t]
L.mtrt_cuda_module_load_from_ptx.restype = ctypes.c_void_p
L.mtrt_cuda_module_get_function.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int64]
L.mtrt_cuda_module_get_function.restype = ctypes.c_void_p
mod = L.mtrt_cuda_module_load_from_ptx(b"", 0)
assert L.mtrt_cuda_module_get_function(mod, b"main_quantize_kernel_0", 22)
assert L.mtrt_cuda_module_get_function(mod, b"main_linear_kernel_3", 20)
print("MANIFEST OK")
"""
    r = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, QL_MTRT_MANIFEST=str(manifest)), capture_output=True, text=True)
    assert r.returncode == 0 and "MANIFEST OK" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
def test_library_kernels_through_the_launch_abi(rt):
    """Kernel names bound to library kernels: same host-side calls, hand-written sm_100a code."""
    mod = rt.mtrt_cuda_module_load_from_ptx(b"", 0)
    g = torch.Generator(device="cpu").manual_seed(9)
    x = torch.randn((64, 256), generator=g).cuda()
    s = (x.abs().max() / 127).reshape(())
    q = torch.empty((64, 256), dtype=torch.int8, device="cuda")
    assert rt.ql_mtrt_bind_kernel(b"quantize_kernel", b"ql:quantize;in=f32;out=i8;scale=f32;shape=64x256") == 0
    fn = rt.mtrt_cuda_module_get_function(mod, b"quantize_kernel", 15)
    stream = torch.cuda.current_stream().cuda_stream
    arr, keep = _args(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(s.data_ptr()), ctypes.c_void_p(q.data_ptr()))
    # grid and block describe the generated kernel the name used to denote; they are ignored
    rt.mtrt_cuda_launch_kernel(fn, 1, 1, 1, 128, 1, 1, 0, stream, arr)
    torch.cuda.synchronize()
    assert rt.mtrt_cuda_last_error() == b""
    want = orc.quantize(x.cpu().numpy(), orc.F32, s.cpu().numpy(), orc.F32, orc.I8)
    assert np.array_equal(q.cpu().numpy(), want)

    # per-channel int8 weights and the W8A16 linear, by self-describing names
    w = (torch.randn((32, 128), generator=g) * 0.02).to(torch.float16).cuda()
    ws = ql.amax_scale(w, ql.int8, dim=0)
    wq = torch.empty((32, 128), dtype=torch.int8, device="cuda")
    name = b"ql:quantize;in=f16;out=i8;scale=f16;shape=32x128;axis=0"
    arr, keep = _args(ctypes.c_void_p(w.data_ptr()), ctypes.c_void_p(ws.data_ptr()), ctypes.c_void_p(wq.data_ptr()))
    rt.mtrt_cuda_launch_kernel(rt.mtrt_cuda_module_get_function(mod, name, len(name)), 1, 1, 1, 1, 1, 1, 0, stream, arr)
    xa = torch.randn((4, 128), generator=g).to(torch.bfloat16).cuda()
    y = torch.empty((4, 32), dtype=torch.bfloat16, device="cuda")
    name = b"ql:linear_w8a16;x=bf16;scale=f16;M=4;N=32;K=128"
    arr, keep = _args(ctypes.c_void_p(xa.data_ptr()), ctypes.c_void_p(wq.data_ptr()), ctypes.c_void_p(ws.data_ptr()), ctypes.c_void_p(y.data_ptr()))
    rt.mtrt_cuda_launch_kernel(rt.mtrt_cuda_module_get_function(mod, name, len(name)), 1, 1, 1, 1, 1, 1, 0, stream, arr)
    torch.cuda.synchronize()
    assert rt.mtrt_cuda_last_error() == b""
    assert torch.equal(wq, ql.quantize(w, ws, ql.int8, 0))
    assert torch.equal(y, ql.linear_w8a16(xa, wq, ws))
    rt.mtrt_cuda_module_unload(mod)


@pytest.mark.gpu
def test_nvfp4_through_the_launch_abi(rt):
    """tensorrt.dynamic_quantize and the block dequantize of its data as library kernels named by their specs."""
    mod = rt.mtrt_cuda_module_load_from_ptx(b"", 0)
    g = torch.Generator(device="cpu").manual_seed(11)
    x = (torch.randn((8, 64), generator=g) * 3).cuda()
    gs = torch.ones((), device="cuda")
    data = torch.empty(8 * 64 // 2, dtype=torch.uint8, device="cuda")
    scales = torch.empty((8, 4), dtype=torch.float8_e4m3fn, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    name = b"ql:dynamic_quantize;in=f32;shape=8x64;axis=1"
    arr, keep = _args(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(gs.data_ptr()), ctypes.c_void_p(data.data_ptr()), ctypes.c_void_p(scales.data_ptr()))
    rt.mtrt_cuda_launch_kernel(rt.mtrt_cuda_module_get_function(mod, name, len(name)), 1, 1, 1, 1, 1, 1, 0, stream, arr)
    torch.cuda.synchronize()
    assert rt.mtrt_cuda_last_error() == b""
    want_q, want_s = orc.dynamic_quantize_nvfp4(x.cpu().numpy(), orc.F32, 1.0)
    assert np.array_equal(data.cpu().numpy().reshape(want_q.shape), want_q)
    assert np.array_equal(scales.view(torch.uint8).cpu().numpy(), want_s)
    # second step: data * f32 block scales
    block_scales = scales.float().contiguous()
    y = torch.empty((8, 64), device="cuda")
    name = b"ql:dequantize;in=f4;out=f32;scale=f32;shape=8x64;scale_shape=8x4"
    arr, keep = _args(ctypes.c_void_p(data.data_ptr()), ctypes.c_void_p(block_scales.data_ptr()), ctypes.c_void_p(y.data_ptr()))
    rt.mtrt_cuda_launch_kernel(rt.mtrt_cuda_module_get_function(mod, name, len(name)), 1, 1, 1, 1, 1, 1, 0, stream, arr)
    torch.cuda.synchronize()
    assert rt.mtrt_cuda_last_error() == b""
    assert np.array_equal(y.cpu().numpy(), orc.dequantize_nvfp4(want_q, want_s, 1.0, orc.F32))
    rt.mtrt_cuda_module_unload(mod)


@pytest.mark.gpu
def test_dynamic_shape_memrefs_through_the_launch_abi(rt):
    """A program compiled with a dynamic batch dimension: each memref with a `?` dimension is followed in `args` by
    that size (and by the strides that depend on it) as i64 values, the way the compiler unpacks memrefs
    (compiler/lib/Passes/1_Core/KernelToCUDA/KernelToCUDA.cpp:94-108).  Same results as the static spelling."""
    mod = rt.mtrt_cuda_module_load_from_ptx(b"", 0)
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device="cpu").manual_seed(21)
    i64, vp = ctypes.c_int64, ctypes.c_void_p
    # quantize f32 [?, 256] -> i8 with rows = 48: args are in, in.size0, scale, out, out.size0
    rows = 48
    x = torch.randn((rows, 256), generator=g).cuda()
    s = (x.abs().max() / 127).reshape(())
    q = torch.empty((rows, 256), dtype=torch.int8, device="cuda")
    name = b"ql:quantize;in=f32;out=i8;scale=f32;shape=?x256"
    arr, keep = _args(vp(x.data_ptr()), i64(rows), vp(s.data_ptr()), vp(q.data_ptr()), i64(rows))
    rt.mtrt_cuda_launch_kernel(rt.mtrt_cuda_module_get_function(mod, name, len(name)), 1, 1, 1, 1, 1, 1, 0, stream, arr)
    torch.cuda.synchronize()
    assert rt.mtrt_cuda_last_error() == b""
    assert torch.equal(q, ql.quantize(x, s, ql.int8))
    # a dynamic inner dimension makes the outer stride dynamic too: [4, ?] passes size1 and then stride0
    x2 = x[:4].contiguous()
    q2 = torch.empty((4, 256), dtype=torch.int8, device="cuda")
    name = b"ql:quantize;in=f32;out=i8;scale=f32;shape=4x?"
    arr, keep = _args(vp(x2.data_ptr()), i64(256), i64(256), vp(s.data_ptr()), vp(q2.data_ptr()), i64(256), i64(256))
    rt.mtrt_cuda_launch_kernel(rt.mtrt_cuda_module_get_function(mod, name, len(name)), 1, 1, 1, 1, 1, 1, 0, stream, arr)
    torch.cuda.synchronize()
    assert rt.mtrt_cuda_last_error() == b"" and torch.equal(q2, q[:4])
    # a stride that is not the dense one is refused, not misread
    arr, keep = _args(vp(x2.data_ptr()), i64(256), i64(512), vp(s.data_ptr()), vp(q2.data_ptr()), i64(256), i64(256))
    rt.mtrt_cuda_launch_kernel(rt.mtrt_cuda_module_get_function(mod, name, len(name)), 1, 1, 1, 1, 1, 1, 0, stream, arr)
    assert b"not dense row-major" in rt.mtrt_cuda_last_error()
    # W8A16 linear with a dynamic number of tokens: x, x.size0, w, scale, y, y.size0
    w = (torch.randn((32, 128), generator=g) * 0.02).to(torch.float16).cuda()
    ws = ql.amax_scale(w, ql.int8, dim=0)
    wq = ql.quantize(w, ws, ql.int8, 0)
    for m in (3, 20):
        xa = torch.randn((m, 128), generator=g).to(torch.bfloat16).cuda()
        y = torch.empty((m, 32), dtype=torch.bfloat16, device="cuda")
        name = b"ql:linear_w8a16;x=bf16;scale=f16;M=?;N=32;K=128"
        arr, keep = _args(vp(xa.data_ptr()), i64(m), vp(wq.data_ptr()), vp(ws.data_ptr()), vp(y.data_ptr()), i64(m))
        rt.mtrt_cuda_launch_kernel(rt.mtrt_cuda_module_get_function(mod, name, len(name)), 1, 1, 1, 1, 1, 1, 0, stream, arr)
        torch.cuda.synchronize()
        assert rt.mtrt_cuda_last_error() == b""
        assert torch.equal(y, ql.linear_w8a16(xa, wq, ws))
    rt.mtrt_cuda_module_unload(mod)
