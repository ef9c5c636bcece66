"""Build ``ramtorch_b200/librt_b200.so`` in-tree with nvcc for sm_100a.

    python -m ramtorch_b200.csrc.build [--force] [--verbose]

The library is plain CUDA C++ behind a C ABI (include/rt_b200.h): no torch headers, no pybind.
It links the shared CUDA runtime so that, inside a PyTorch process, it uses the runtime
instance torch already loaded (same primary contexts, streams and current device).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
ROOT = os.path.dirname(PKG)
OUT = os.path.join(PKG, "librt_b200.so")
SOURCES = ["adamw_sr.cu", "offload.cu"]
DEPS = SOURCES + ["philox.cuh", "rt_internal.h", os.path.join(ROOT, "include", "rt_b200.h")]


def nvcc_path() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if os.path.exists(cand):
        return cand
    found = shutil.which("nvcc")
    if not found:
        raise RuntimeError("nvcc not found: librt_b200.so cannot be built")
    return found


def stale() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    return any(os.path.getmtime(os.path.join(HERE, d)) > t for d in DEPS)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not stale():
        return OUT
    nvcc = nvcc_path()
    cuda_lib = os.path.join(os.path.dirname(os.path.dirname(nvcc)), "lib64")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "-Xcompiler", "-fPIC,-O2,-Wall", "-shared", "-cudart", "shared",
           "-Xlinker", f"-rpath={cuda_lib}", "-o", OUT + ".tmp"]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(HERE, s) for s in SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building librt_b200.so")
    os.replace(OUT + ".tmp", OUT)
    return OUT


FASTSCAN_SRC = os.path.join(HERE, "fastscan.cpp")
FASTSCAN_OUT = os.path.join(PKG, "_fastscan.so")


def build_fastscan(force: bool = False) -> str:
    """Build ``ramtorch_b200/_fastscan.so``, the host-side helper that walks long parameter lists in
    C++ (g++ against the torch headers of the running interpreter).  It only reads tensor pointers
    and properties; the optimizer works without it, with per-tensor Python passes instead."""
    if not force and os.path.exists(FASTSCAN_OUT) and os.path.getmtime(FASTSCAN_OUT) >= os.path.getmtime(FASTSCAN_SRC):
        return FASTSCAN_OUT
    import sysconfig

    import torch
    from torch.utils import cpp_extension as ce
    gxx = shutil.which("g++")
    if not gxx:
        raise RuntimeError("g++ not found: _fastscan.so cannot be built")
    inc = ce.include_paths() + [sysconfig.get_paths()["include"]]
    libs = ce.library_paths()
    cmd = [gxx, "-O2", "-std=c++17", "-shared", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           "-DTORCH_EXTENSION_NAME=_fastscan", "-DTORCH_API_INCLUDE_EXTENSION_H"]
    cmd += [f"-I{i}" for i in inc] + [FASTSCAN_SRC, "-o", FASTSCAN_OUT + ".tmp"]
    cmd += [f"-L{d}" for d in libs] + [f"-Wl,-rpath,{d}" for d in libs] + ["-ltorch_python", "-ltorch", "-ltorch_cpu", "-lc10"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("g++ failed building _fastscan.so")
    os.replace(FASTSCAN_OUT + ".tmp", FASTSCAN_OUT)
    return FASTSCAN_OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    print(build_fastscan(force="--force" in sys.argv))
