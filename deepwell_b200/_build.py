"""Builds the C-ABI shared library (CUDA kernels for sm_100a) in-tree with nvcc.

    python deepwell_b200/_build.py [--force] [--verbose]      (or: python -m deepwell_b200._build)

The file imports nothing from the package, so it can be run (or loaded by path) while the library
is missing or stale.

Outputs: deepwell_b200/lib/libdw_mxfp8.so (the product: kernels + C ABI; nvcc cross-compiles without
a GPU) and deepwell_b200/_C.so (csrc/python_bindings.cpp: the torch-tensor layer over that C ABI,
compiled with g++ against the installed torch headers and linked to the library by a relative rpath).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

_PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_PKG, "csrc")
LIB_DIR = os.path.join(_PKG, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libdw_mxfp8.so")
SOURCES = ["mx_quantize.cu", "mx_gemm.cu", "dw_abi.cu"]
HEADERS = ["dw_common.cuh", "dw_ptx.cuh", os.path.join("..", "..", "include", "dw_mxfp8.h")]
EXT_PATH = os.path.join(_PKG, "_C.so")
EXT_SOURCE = os.path.join(CSRC, "python_bindings.cpp")


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or add it to PATH")


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not is_stale():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [
        nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
        "-shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
        "-DDW_BUILDING_LIB", "-o", LIB_PATH,
    ]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(CSRC, s) for s in SOURCES]
    # the environment's CC may point at a compiler nvcc cannot drive; use the system g++
    env = dict(os.environ)
    env.pop("CC", None); env.pop("CXX", None)
    res = subprocess.run(cmd, env=env, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libdw_mxfp8.so")
    return LIB_PATH


def ext_is_stale() -> bool:
    if not os.path.exists(EXT_PATH):
        return True
    t = os.path.getmtime(EXT_PATH)
    deps = [EXT_SOURCE, os.path.join(_PKG, "..", "include", "dw_mxfp8.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build_ext(force: bool = False, verbose: bool = False) -> str:
    """Compiles csrc/python_bindings.cpp into deepwell_b200/_C.so (needs libdw_mxfp8.so to link against)."""
    build(force=False, verbose=verbose)
    if not force and not ext_is_stale():
        return EXT_PATH
    import sysconfig

    import torch
    from torch.utils import cpp_extension as ce
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_home = ce.CUDA_HOME or "/usr/local/cuda"
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-DTORCH_EXTENSION_NAME=_C",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch.compiled_with_cxx11_abi())}"]
    for inc in ce.include_paths() + [sysconfig.get_paths()["include"], os.path.join(cuda_home, "include")]:
        cmd += ["-isystem", inc]
    cmd += [EXT_SOURCE, "-o", EXT_PATH, "-L", torch_lib, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
            "-ltorch_python", "-L", LIB_DIR, "-ldw_mxfp8", "-Wl,-rpath,$ORIGIN/lib", f"-Wl,-rpath,{torch_lib}"]
    env = dict(os.environ)
    env.pop("CC", None); env.pop("CXX", None)
    res = subprocess.run(cmd, env=env, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("g++ failed building deepwell_b200/_C.so")
    return EXT_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    print(build_ext(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
