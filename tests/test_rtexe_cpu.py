"""The compiled-executable reader (ql_rtexe_*): data segments of a `.rtexe` file (FlatBuffers, schema
executor/include/mlir-executor/Runtime/API/Executable.fbs of the reference), and loading a module's PTX straight out
of one through the launch ABI.  The files are written by tests/rtexe_writer.py; parsing needs no GPU."""
import ctypes
import os

import pytest

from conftest import ROOT
from qlinear import _lib
from rtexe_writer import build_rtexe

PTX = open(os.path.join(ROOT, "tests", "golden", "add_scalar.ptx"), "rb").read()


class SegInfo(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char_p), ("data", ctypes.c_void_p), ("size", ctypes.c_uint64), ("uninitialized_size", ctypes.c_uint64),
                ("alignment", ctypes.c_uint32), ("constant", ctypes.c_int32), ("address_space", ctypes.c_int32), ("kind", ctypes.c_int32)]


@pytest.fixture(scope="module")
def L():
    lib = ctypes.CDLL(_lib.LIB_PATH)
    vp = ctypes.c_void_p
    lib.ql_rtexe_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
    lib.ql_rtexe_open_memory.argtypes = [ctypes.c_char_p, ctypes.c_uint64, ctypes.POINTER(vp)]
    lib.ql_rtexe_close.argtypes = [vp]
    lib.ql_rtexe_name.argtypes = [vp]
    lib.ql_rtexe_name.restype = ctypes.c_char_p
    lib.ql_rtexe_num_segments.argtypes = [vp]
    lib.ql_rtexe_segment.argtypes = [vp, ctypes.c_int32, ctypes.POINTER(SegInfo)]
    lib.ql_rtexe_find_segment.argtypes = [vp, ctypes.c_char_p]
    lib.ql_last_error.restype = ctypes.c_char_p
    lib.mtrt_cuda_module_load_from_ptx_file.argtypes = [ctypes.c_char_p, ctypes.c_size_t]
    lib.mtrt_cuda_module_load_from_ptx_file.restype = vp
    lib.mtrt_cuda_module_get_function.argtypes = [vp, ctypes.c_char_p, ctypes.c_int64]
    lib.mtrt_cuda_module_get_function.restype = vp
    lib.mtrt_cuda_module_unload.argtypes = [vp]
    lib.mtrt_cuda_last_error.restype = ctypes.c_char_p
    return lib


SEGMENTS = [
    {"name": "weights_0", "data": bytes(range(200)), "alignment": 256, "constant": True, "address_space": 2},
    {"name": "main_kernels_ptx", "data": PTX, "alignment": 16, "constant": True, "address_space": 0},
    {"name": "scratch", "data": b"", "alignment": 64, "constant": False, "address_space": 2, "uninitialized_size": 4096},
    {"name": "a_cubin", "data": b"\x7fELF" + b"\x00" * 60, "alignment": 16, "constant": True, "address_space": 0},
]


def test_segments_are_read_back(L, tmp_path):
    blob = build_rtexe("program_main", SEGMENTS)
    path = tmp_path / "program.rtexe"
    path.write_bytes(blob)
    exe = ctypes.c_void_p()
    assert L.ql_rtexe_open(str(path).encode(), ctypes.byref(exe)) == 0, L.ql_last_error()
    assert L.ql_rtexe_name(exe) == b"program_main"
    assert L.ql_rtexe_num_segments(exe) == len(SEGMENTS)
    kinds = []
    for i, s in enumerate(SEGMENTS):
        info = SegInfo()
        assert L.ql_rtexe_segment(exe, i, ctypes.byref(info)) == 0
        assert info.name == s["name"].encode() and info.size == len(s["data"])
        assert info.alignment == s["alignment"] and info.constant == int(s["constant"]) and info.address_space == s["address_space"]
        assert info.uninitialized_size == s.get("uninitialized_size", 0)
        if s["data"]:
            assert ctypes.string_at(info.data, info.size) == s["data"]
        kinds.append(info.kind)
    assert kinds == [0, 1, 0, 2]   # data, PTX, data, cubin
    assert L.ql_rtexe_find_segment(exe, b"main_kernels_ptx") == 1 and L.ql_rtexe_find_segment(exe, b"nope") == -1
    assert L.ql_rtexe_segment(exe, 9, ctypes.byref(SegInfo())) != 0
    L.ql_rtexe_close(exe)


def test_damaged_files_are_refused(L):
    blob = build_rtexe("p", SEGMENTS)
    exe = ctypes.c_void_p()
    for bad in (blob[:40], b"\xff" * 64, blob[:len(blob) - len(PTX) // 2], b""):
        assert L.ql_rtexe_open_memory(bad, len(bad), ctypes.byref(exe)) != 0
        assert b"rtexe" in L.ql_last_error()
    # every truncation either parses consistently or is refused; none crashes
    for cut in range(0, len(blob), max(1, len(blob) // 97)):
        if L.ql_rtexe_open_memory(blob[:cut], cut, ctypes.byref(exe)) == 0:
            L.ql_rtexe_close(exe)


def test_module_bytes_come_straight_out_of_an_executable(L, tmp_path):
    path = tmp_path / "program.rtexe"
    path.write_bytes(build_rtexe("program_main", SEGMENTS))
    spec = f"{path}#main_kernels_ptx".encode()
    mod = L.mtrt_cuda_module_load_from_ptx_file(spec, len(spec))
    assert mod, L.mtrt_cuda_last_error()
    # library kernels resolve by name without a GPU; the caller's own kernels are JIT-compiled from the segment's PTX
    name = b"ql:quantize;in=f32;out=i8;scale=f32;shape=16"
    assert L.mtrt_cuda_module_get_function(mod, name, len(name))
    L.mtrt_cuda_module_unload(mod)
    missing = f"{path}#no_such_segment".encode()
    assert not L.mtrt_cuda_module_load_from_ptx_file(missing, len(missing))
    assert b"no data segment" in L.mtrt_cuda_last_error()


@pytest.mark.gpu
def test_kernel_from_an_executable_runs(L, tmp_path):
    import torch
    path = tmp_path / "program.rtexe"
    path.write_bytes(build_rtexe("program_main", SEGMENTS))
    spec = f"{path}#main_kernels_ptx".encode()
    mod = L.mtrt_cuda_module_load_from_ptx_file(spec, len(spec))
    fn = L.mtrt_cuda_module_get_function(mod, b"add_scalar", 10)
    assert fn, L.mtrt_cuda_last_error()
    L.mtrt_cuda_launch_kernel.argtypes = [ctypes.c_void_p] + [ctypes.c_int32] * 7 + [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p)]
    n = 300
    x = torch.arange(n, dtype=torch.float32, device="cuda")
    holders = [ctypes.c_void_p(x.data_ptr()), ctypes.c_int32(n), ctypes.c_float(4.0)]
    arr = (ctypes.c_void_p * 3)(*[ctypes.cast(ctypes.byref(h), ctypes.c_void_p) for h in holders])
    L.mtrt_cuda_launch_kernel(fn, (n + 63) // 64, 1, 1, 64, 1, 1, 0, torch.cuda.current_stream().cuda_stream, arr)
    torch.cuda.synchronize()
    assert torch.equal(x.cpu(), torch.arange(n, dtype=torch.float32) + 4.0)
    L.mtrt_cuda_module_unload(mod)
