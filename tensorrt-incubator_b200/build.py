"""Builds lib/libqlinear_b200.so from csrc/*.cu with nvcc for sm_100a (and nothing else).

Run as a script or call build().  The shared library links the CUDA runtime statically and
resolves driver entry points at run time, so it loads on a machine without a GPU or driver
(compute calls then fail with QL_ERR_NO_DEVICE).
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "lib", "libqlinear_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr",
    "-I", os.path.join(ROOT, "include"), "-I", CSRC,
]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA extension cannot be built")


def _newer(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(os.path.dirname(LIB), exist_ok=True)
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    headers = sorted(glob.glob(os.path.join(CSRC, "*.cuh"))) + sorted(glob.glob(os.path.join(ROOT, "include", "*.h")))
    nvcc = _nvcc()
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    jobs = []
    objs = []
    for src in sources:
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if force or not _newer(obj, [src] + headers):
            cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, env=env, capture_output=True, text=True)
        if verbose or r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(run, jobs))
    if jobs or force or not _newer(LIB, objs):
        run([nvcc, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-ldl"])
    return LIB


TVMFFI_LIB = os.path.join(HERE, "lib", "libqlinear_b200_tvmffi.so")


def build_tvm_ffi_plugin(force: bool = False):
    """The TVM-FFI plug-in library (csrc_tvmffi/), built only where the tvm_ffi package is installed.
    It links libqlinear_b200.so and libtvm_ffi.so; returns its path or None."""
    try:
        import tvm_ffi
    except Exception:
        return None
    root = os.path.dirname(tvm_ffi.__file__)
    inc, libdir = os.path.join(root, "include"), os.path.join(root, "lib")
    src = os.path.join(HERE, "csrc_tvmffi", "ql_tvm_ffi.cc")
    if not (os.path.exists(os.path.join(inc, "tvm", "ffi", "c_api.h")) and os.path.exists(os.path.join(libdir, "libtvm_ffi.so"))):
        return None
    if not force and _newer(TVMFFI_LIB, [src, LIB, os.path.join(ROOT, "include", "qlinear_b200.h")]):
        return TVMFFI_LIB
    gxx = shutil.which("g++") or "g++"
    cmd = [gxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-I", inc, "-I", os.path.join(ROOT, "include"),
           src, "-o", TVMFFI_LIB, "-L", os.path.dirname(LIB), "-lqlinear_b200", "-L", libdir, "-ltvm_ffi",
           "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + libdir]
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    r = subprocess.run(cmd, env=env, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("building the TVM-FFI plug-in failed:\n" + r.stdout + r.stderr)
    return TVMFFI_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_tvm_ffi_plugin(force="--force" in sys.argv))
