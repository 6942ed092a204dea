"""Ahead-of-time build of libavefp4.so (hand-written CUDA for sm_100a) with nvcc.

The reference compiles its launcher with gcc at first use
(python/avelang/backends/nvidia/driver.py:325-333, python/avelang/runtime/build.py:16-56);
here the kernels are fixed, so the library is built once, in-tree, next to this file.
"""
from __future__ import annotations

import os
import shutil
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
LIB_PATH = os.path.join(_HERE, "libavefp4.so")
SOURCES = ["ave_fp4_api.cu"]
HEADERS = ["sm100_ptx.cuh", "gemm_fp4_sm100.cuh", "gemm_fp4_skinny_sm100.cuh", "quantize_fp4.cuh"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or add it to PATH")


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS]
    deps.append(os.path.join(_HERE, "..", "include", "ave_fp4.h"))
    return any(os.path.getmtime(d) > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if it is missing or older than its sources; return its path."""
    if not force and not is_stale():
        return LIB_PATH
    cmd = [_nvcc(), *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", LIB_PATH, *[os.path.join(CSRC, s) for s in SOURCES]]
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout)
    if verbose:
        print(proc.stdout)
    return LIB_PATH


SHIM_SRC = os.path.join(_HERE, "..", "python", "src", "avefp4_shim.cc")
SHIM_DIR = os.path.join(_HERE, "..", "python", "avelang_kernels")


def shim_path() -> str:
    import sysconfig

    return os.path.join(SHIM_DIR, "_avefp4_shim" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))


def build_shim(force: bool = False) -> str:
    """Compile python/src/avefp4_shim.cc (the pybind11 module over the C ABI) next to python/avelang_kernels,
    linked against libavefp4.so through an rpath relative to the module.  The reference builds its native module
    from the same directory with CMake (python/CMakeLists.txt:19); one g++ call is enough for a shim."""
    import sysconfig

    import pybind11

    out = shim_path()
    build()
    if not force and os.path.exists(out) and os.path.getmtime(out) >= max(os.path.getmtime(SHIM_SRC),
                                                                        os.path.getmtime(os.path.join(_HERE, "..", "include", "ave_fp4.h"))):
        return out
    cxx = shutil.which("g++") or "/usr/bin/g++"
    cmd = [cxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-I", pybind11.get_include(), "-I",
           sysconfig.get_paths()["include"], SHIM_SRC, "-L", _HERE, "-lavefp4", "-Wl,-rpath,$ORIGIN/../../avelang_b200", "-o", out]
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError("building the pybind11 shim failed:\n" + proc.stdout)
    return out


if __name__ == "__main__":
    print(build(force=True, verbose=True))
    print(build_shim(force=True))
