"""The C-ABI shared library on a machine without a GPU: it loads, exports every symbol the
headers declare, validates arguments with the reference verifier's wording, and refuses to
compute without a device (there is no CPU path in the product)."""
import ctypes
import os
import re

import pytest
import torch

from conftest import ROOT

import qlinear
from qlinear import _lib


def _declared_symbols():
    names = []
    for fn in sorted(os.listdir(os.path.join(ROOT, "include"))):
        text = open(os.path.join(ROOT, "include", fn)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        text = "\n".join(l for l in text.splitlines() if not l.lstrip().startswith("#"))
        names += re.findall(r"(?:QL_API|MTRT_CAPI_EXPORTED)\s+[\w\s\*]*?\b(\w+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    L = ctypes.CDLL(_lib.LIB_PATH)
    names = _declared_symbols()
    assert len(names) >= 12
    for n in names:
        assert hasattr(L, n), n
    assert set(_lib.SIGNATURES) <= set(names)
    assert _lib.lib().ql_version() >= 100


def _t(dtype, shape, ptr=0x1000):
    return _lib.make_tensor(ptr, dtype, shape)


def _err(rc):
    assert rc != 0
    return _lib.lib().ql_last_error().decode()


@pytest.mark.parametrize("fn", ["ql_quantize", "ql_dequantize"])
def test_verifier_messages(fn):
    """Wording of tensorrt/lib/TensorRT/IR/Verification.cpp:1182-1265 / 1296-1380."""
    L = _lib.lib()
    f = getattr(L, fn)
    is_q = fn == "ql_quantize"

    def call(data_shape, scale_shape, qdtype=_lib.I8, axis=None):
        fl, q, s = _t(_lib.F32, data_shape), _t(qdtype, data_shape), _t(_lib.F32, scale_shape)
        a = _lib.make_attrs(axis)
        return f(fl, s, q, a, None) if is_q else f(q, s, fl, a, None)

    assert "axis value must be provided" in _err(call([4, 4], [4]))
    assert "expected axis to be non-negative and less than 2" in _err(call([4, 4], [4], axis=2))
    assert "expected the scales tensor dimension to match" in _err(call([4, 4], [3], axis=0))
    assert "axis value shouldn't be provided" in _err(call([4, 4], [], axis=0))
    assert "Scale value must be scalar for per-tensor" in _err(call([2, 4, 4], [2, 2]))
    assert "Block quantization is supported only for int4, fp4 or fp8" in _err(call([4, 4], [2, 4]))
    assert "Axis is not valid in this case" in _err(call([4, 4], [2, 4], _lib.I4, axis=0))
    assert "blocking dimension should be either last or second last" in _err(call([4, 4, 4], [2, 4, 4], _lib.I4))
    assert "all input and scale dimensions match except a single blocking dimension" in _err(call([4, 4], [2, 2], _lib.I4))


def test_type_rules():
    L = _lib.lib()
    a = _lib.make_attrs()
    rc = L.ql_quantize(_t(_lib.I8, [4]), _t(_lib.F32, []), _t(_lib.I8, [4]), a, None)
    assert "valid conversions are" in _err(rc)
    rc = L.ql_dequantize(_t(_lib.F32, [4]), _t(_lib.F32, []), _t(_lib.F32, [4]), a, None)
    assert "valid conversions are" in _err(rc)
    rc = L.ql_quantize(_t(_lib.F32, [4]), _t(_lib.F32, []), _t(_lib.I8, [5]), a, None)
    assert "shapes differ" in _err(rc)
    rc = L.ql_quantize(_t(_lib.F32, [4]), _t(_lib.I8, []), _t(_lib.I8, [4]), a, None)
    assert "scale must be f32, f16 or bf16" in _err(rc)
    rc = L.ql_quantize(None, _t(_lib.F32, []), _t(_lib.I8, [4]), a, None)
    assert "is null" in _err(rc)


def test_linear_argument_rules():
    L = _lib.lib()
    x, w, y = _t(_lib.BF16, [4, 128]), _t(_lib.I8, [32, 128]), _t(_lib.BF16, [4, 32])
    assert "expected the scales tensor dimension to match" in _err(L.ql_linear_w8a16(x, w, _t(_lib.F32, [31]), y, None))
    assert "x and y must both be f16 or both be bf16" in _err(L.ql_linear_w8a16(_t(_lib.F32, [4, 128]), w, _t(_lib.F32, [32]), y, None))
    assert "y must be [M,N]" in _err(L.ql_linear_w8a16(x, w, _t(_lib.F32, [32]), _t(_lib.BF16, [4, 33]), None))
    w4 = _t(_lib.I4, [32, 128])
    assert "single blocking dimension" in _err(L.ql_linear_w4a16(x, w4, _t(_lib.F32, [32, 3]), y, None))
    assert "multiples of 128" in _err(L.ql_linear_w4a16(x, w4, _t(_lib.F32, [32, 2]), y, None))


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-device behaviour")
def test_no_cpu_fallback():
    """Without a GPU the product refuses to compute instead of falling back."""
    x = torch.ones(4)
    with pytest.raises(_lib.QlError) as e:
        qlinear.quantize(x, 1.0, qlinear.int8)
    assert e.value.status == _lib.ERR_NO_DEVICE
    # and the raw entry point reports a CUDA failure rather than computing on the host
    buf = (ctypes.c_float * 64)()
    out = (ctypes.c_int8 * 64)()
    sc = (ctypes.c_float * 1)(1.0)
    p = lambda b: ctypes.cast(b, ctypes.c_void_p).value
    rc = _lib.lib().ql_quantize(_t(_lib.F32, [64], p(buf)), _t(_lib.F32, [], p(sc)), _t(_lib.I8, [64], p(out)), _lib.make_attrs(), None)
    assert rc in (_lib.ERR_NO_DEVICE, _lib.ERR_CUDA)
    assert bytes(out) == bytes(64)


def _peer(world=2, rank=0, base=0x10000, with_all=True):
    b = _lib.QlPeerBuffer()
    for r in range(min(world, _lib.QL_MAX_PEERS)):
        b.replica[r] = base + r * 0x100000
    b.all = 0x9000000 if with_all else None
    b.world, b.rank = world, rank
    return b


def test_peer_entry_points_validate_before_touching_a_device():
    """Argument rules of the fused GEMM + collective path (no reference counterpart)."""
    L = _lib.lib()
    xq, wq = _t(_lib.F8E4M3, [256, 128]), _t(_lib.F8E4M3, [512, 128])
    sx, sw = _t(_lib.F32, []), _t(_lib.F32, [])
    ok = _peer()
    assert "bad world / rank" in _err(L.ql_gemm_fp8_peer(xq, wq, sx, sw, _peer(world=9), _lib.BF16, 512, 0, _lib.PEER_STORE_ALL, None))
    assert "unknown peer mode" in _err(L.ql_gemm_fp8_peer(xq, wq, sx, sw, ok, _lib.BF16, 512, 0, 7, None))
    assert "smaller than N" in _err(L.ql_gemm_fp8_peer(xq, wq, sx, sw, ok, _lib.BF16, 256, 0, _lib.PEER_STORE_ALL, None))
    assert "no address for this mode" in _err(L.ql_gemm_fp8_peer(xq, wq, sx, sw, _peer(with_all=False), _lib.BF16, 512, 0, _lib.PEER_ADD_ALL, None))
    assert "offset % 8 == 0" in _err(L.ql_gemm_fp8_peer(xq, wq, sx, sw, ok, _lib.BF16, 512, 4, _lib.PEER_STORE_ALL, None))
    wq_odd = _t(_lib.F8E4M3, [520, 128])
    assert "N % 32 == 0" in _err(L.ql_gemm_fp8_peer(xq, wq_odd, sx, sw, ok, _lib.BF16, 1024, 0, _lib.PEER_ADD_ALL, None))
    # owner blocks must be whole 128-row tiles
    assert "multiple of 128 x world" in _err(L.ql_gemm_fp8_peer(_t(_lib.F8E4M3, [384, 128]), wq, sx, sw, _peer(world=2), _lib.BF16, 512, 0,
                                                                 _lib.PEER_ADD_OWNER, None))
    assert "replica 1 has no address" in _err(L.ql_peer_barrier(_missing_replica(), None))
    assert "multiples of 16 bytes" in _err(L.ql_peer_broadcast(ok, 8, 64, None))
    assert "must be bf16 or f16" in _err(L.ql_peer_reduce(ok, _lib.F32, 0, 64, None))
    assert "no replication address" in _err(L.ql_peer_reduce(_peer(with_all=False), _lib.BF16, 0, 64, None))


def test_nccl_entry_points_validate_their_arguments():
    """The NCCL module of the C ABI (executor/lib/Runtime/Backend/Lua/Modules/NCCL/NCCLModule.cpp:233-385): argument
    rules that need neither a GPU nor a communicator."""
    import ctypes
    L = _lib.lib()
    none = ctypes.c_void_p()
    assert "not a communicator" in _err(L.ql_nccl_all_reduce(None, None, None, 4, _lib.F32, 0, None))
    assert "not a communicator" in _err(L.ql_nccl_all_gather(None, None, None, 4, None))
    assert "not a communicator" in _err(L.ql_nccl_comm_split(None, 0, 0, ctypes.byref(none)))
    assert "not a communicator" in _err(L.ql_nccl_comm_rank(None, None, None))
    assert L.ql_nccl_comm_destroy(None) == 0           # destroying nothing is not an error
    uid = ctypes.create_string_buffer(128)
    rc = L.ql_nccl_comm_init_rank(3, 2, 0, uid, 0, ctypes.byref(none))
    assert "rank 3 of 2" in _err(rc)
    assert "null argument" in _err(L.ql_nccl_comm_init_rank(0, 1, 0, None, 0, ctypes.byref(none)))
    assert "null argument" in _err(L.ql_nccl_unique_id(None))


def _missing_replica():
    b = _peer(world=2)
    b.replica[1] = None
    return b


def test_nvfp4_entry_points_use_the_verifier_wording():
    """tensorrt/lib/TensorRT/IR/Verification.cpp:1270-1290."""
    L = _lib.lib()
    x, gs = _t(_lib.F32, [4, 32]), _t(_lib.F32, [])
    q, s = _t(_lib.F4E2M1, [4, 32]), _t(_lib.F8E4M3, [4, 2])
    assert "currently only block size of 16 is supported!" in _err(L.ql_dynamic_quantize(x, gs, 1, 32, q, s, None))
    assert "invalid axis! Axis can be either last or second last dimension of the input." in _err(
        L.ql_dynamic_quantize(_t(_lib.F32, [2, 4, 32]), gs, 0, 16, _t(_lib.F4E2M1, [2, 4, 32]), _t(_lib.F8E4M3, [2, 4, 2]), None))
    assert "shape(input)[axis] must be divisible by 16." in _err(
        L.ql_dynamic_quantize(_t(_lib.F32, [4, 24]), gs, 1, 16, _t(_lib.F4E2M1, [4, 24]), _t(_lib.F8E4M3, [4, 1]), None))
    assert "second last dimension are not built" in _err(L.ql_dynamic_quantize(_t(_lib.F32, [32, 32]), gs, 0, 16, q, s, None))
    assert "one entry per block of 16" in _err(L.ql_dynamic_quantize(x, gs, 1, 16, q, _t(_lib.F8E4M3, [4, 4]), None))
    assert "rank-0" in _err(L.ql_dynamic_quantize(x, _t(_lib.F32, [1]), 1, 16, q, s, None))
    assert "data must be f4E2M1FN and scales f8E4M3FN" in _err(L.ql_dequantize_nvfp4(_t(_lib.I4, [4, 32]), s, gs, x, None))


def test_nvfp4_axis_and_rank_are_checked_before_any_shape_is_read():
    L = _lib.lib()
    gs = _t(_lib.F32, [])
    q, s = _t(_lib.F4E2M1, [32]), _t(_lib.F8E4M3, [2])
    # a vector with axis -1, a scalar with axis 0 or -1, a rank beyond the structure's capacity
    assert "invalid axis!" in _err(L.ql_dynamic_quantize(_t(_lib.F32, [32]), gs, -1, 16, q, s, None))
    assert "invalid axis!" in _err(L.ql_dynamic_quantize(_t(_lib.F32, []), gs, 0, 16, q, s, None))
    assert "invalid axis!" in _err(L.ql_dynamic_quantize(_t(_lib.F32, []), gs, -1, 16, q, s, None))
    bad = _t(_lib.F32, [32])
    bad.rank = 9
    assert "rank 9" in _err(L.ql_dynamic_quantize(bad, gs, 8, 16, q, s, None))
    # tensorrt.dequantize of f4 data checks the data tensor like every other argument
    f4 = _t(_lib.F4E2M1, [4, 32], ptr=0)
    assert "no data pointer" in _err(L.ql_dequantize(f4, _t(_lib.F8E4M3, [4, 2]), _t(_lib.F32, [4, 32]), _lib.make_attrs(None), None))
    f4 = _t(_lib.F4E2M1, [4, 32])
    f4.rank = 11
    assert "rank 11" in _err(L.ql_dequantize(f4, _t(_lib.F8E4M3, [4, 2]), _t(_lib.F32, [4, 32]), _lib.make_attrs(None), None))


def test_linear_and_matmul_argument_rules():
    """tp.matmul wants operands of one float type (tripy/nvtripy/frontend/ops/matmul.py:31-34); the shapes are those of
    tensorrt.matrix_multiply.  All of it is checked before a device is touched."""
    L = _lib.lib()
    x, w, y = _t(_lib.F32, [3, 4]), _t(_lib.F32, [2, 4]), _t(_lib.F32, [3, 2])
    assert "result of their own type" in _err(L.ql_linear(x, w, None, None, None, _t(_lib.BF16, [3, 2]), None))
    assert "inner dimensions differ" in _err(L.ql_linear(x, _t(_lib.F32, [2, 5]), None, None, None, y, None))
    assert "unexpected operand types" in _err(L.ql_linear(x, _t(_lib.F16, [2, 4]), None, None, None, y, None))
    assert "operands must be f32, f16, bf16, e4m3 or int8" in _err(L.ql_linear(_t(_lib.I4, [3, 4]), _t(_lib.I4, [2, 4]), None, None, None, y, None))
    assert "bias must be a float vector" in _err(L.ql_linear(x, w, None, None, _t(_lib.F32, [3]), y, None))
    assert "scalar or one value per row" in _err(L.ql_linear(x, w, _t(_lib.F32, [2]), None, None, y, None))
    assert "y must be [M,N]" in _err(L.ql_linear(x, w, None, None, None, _t(_lib.F32, [3, 3]), None))
    a, b, c = _t(_lib.F32, [2, 3, 4]), _t(_lib.F32, [1, 4, 5]), _t(_lib.F32, [2, 3, 5])
    assert "share one of f32, f16, bf16" in _err(L.ql_matmul(a, _t(_lib.F16, [1, 4, 5]), c, None))
    assert "equal ranks >= 2" in _err(L.ql_matmul(_t(_lib.F32, [4]), _t(_lib.F32, [4]), _t(_lib.F32, []), None))
    assert "does not give" in _err(L.ql_matmul(a, _t(_lib.F32, [1, 5, 5]), c, None))
    assert "does not broadcast" in _err(L.ql_matmul(a, _t(_lib.F32, [3, 4, 5]), c, None))
    # a mixed broadcast is left to the caller to expand
    assert "all equal to the result's or all 1" in _err(
        L.ql_matmul(_t(_lib.F32, [2, 1, 3, 4]), _t(_lib.F32, [2, 6, 4, 5]), _t(_lib.F32, [2, 6, 3, 5]), None))
    # empty products are no-ops even without a device
    assert L.ql_matmul(_t(_lib.F32, [0, 3, 4]), _t(_lib.F32, [0, 4, 5]), _t(_lib.F32, [0, 3, 5]), None) == 0


def test_emitc_wrappers_compile_as_c_and_link(tmp_path):
    """The `_cwrapper` inlines of the launch-ABI header (C/CUDAModule.h:130-205 of the reference), used from plain C
    the way EmitC-generated host code uses them, compiled and linked against the library (never run)."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None or not os.path.exists("/usr/local/cuda/include/cuda.h"):
        pytest.skip("needs gcc and the CUDA headers")
    src = os.path.join(ROOT, "tests", "golden", "emitc_host_stub.c")
    out = str(tmp_path / "libemitc_stub.so")
    env = {k: v for k, v in os.environ.items() if k not in ("CC", "CXX")}
    r = subprocess.run([gcc, "-std=c11", "-Wall", "-Werror", "-shared", "-fPIC", "-I", os.path.join(ROOT, "include"), "-I", "/usr/local/cuda/include",
                        src, "-o", out, "-L", os.path.dirname(_lib.LIB_PATH), "-lqlinear_b200", "-Wl,--no-undefined", "-Wl,-rpath," + os.path.dirname(_lib.LIB_PATH)],
                       capture_output=True, text=True, env=env)
    assert r.returncode == 0, r.stderr
    text = open(os.path.join(ROOT, "include", "mtrt_cuda_module.h")).read()
    wrappers = set(re.findall(r"\b(mtrt_cuda_\w+)_cwrapper\s*\(", text))
    assert len(wrappers) == 18 and wrappers <= set(_declared_symbols())
