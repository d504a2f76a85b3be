"""Ahead-of-time build of ``libkm_b200.so`` (the C-ABI library) for sm_100a with nvcc.

One fixed build: no per-configuration JIT and no autotuning (the reference compiles one
extension per op and define set at run time, kernel_matmul/compile.py:49-125).  The library is
built in-tree next to this file; it has no dependency on PyTorch or Python.

Usage:  python kernel_matmul_b200/build.py [--force] [--verbose]
(run as a script: importing the package itself requires the built library)
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libkm_b200.so")
HEADER = os.path.join(os.path.dirname(HERE), "include", "km_b200.h")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
]


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _deps() -> list[str]:
    return [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [HEADER, os.path.abspath(__file__)]


def up_to_date() -> bool:
    if not os.path.exists(LIB):
        return False
    t = os.path.getmtime(LIB)
    return all(os.path.getmtime(d) <= t for d in _deps())


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _compile(src: str, verbose: bool) -> str:
    obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
    newest = max(os.path.getmtime(d) for d in _deps() if not d.endswith(".cu") or d == src)
    if os.path.exists(obj) and os.path.getmtime(obj) >= newest:
        return obj
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", src, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}")
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every ``csrc/*.cu`` and link ``libkm_b200.so``; returns its path."""
    if not force and up_to_date():
        return LIB
    os.makedirs(OBJ_DIR, exist_ok=True)
    if force:
        for f in os.listdir(OBJ_DIR):
            if f.endswith(".o"):
                os.remove(os.path.join(OBJ_DIR, f))
    with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose), sources()))
    # The CUDA runtime is linked statically: the library is self-contained and shares the
    # primary context (and therefore streams and allocations) with whatever else is loaded.
    cmd = [_nvcc(), "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
           "-cudart", "static", "-Xlinker", "-soname=libkm_b200.so"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("link of libkm_b200.so failed")
    return LIB


TORCH_SRC = os.path.join(HERE, "csrc_torch", "km_torch.cpp")
TORCH_EXT = os.path.join(HERE, "_C.so")


def build_torch_extension(force: bool = False) -> str:
    """Compile ``csrc_torch/km_torch.cpp`` into ``kernel_matmul_b200/_C.so``: the PyTorch C++
    extension over the C ABI (needs the PyTorch headers of the running interpreter and g++; no
    GPU).  It links against ``libkm_b200.so`` next to it (rpath ``$ORIGIN``)."""
    build()
    deps = [TORCH_SRC, HEADER, LIB, os.path.abspath(__file__)]
    if not force and os.path.exists(TORCH_EXT) and all(os.path.getmtime(d) <= os.path.getmtime(TORCH_EXT) for d in deps):
        return TORCH_EXT
    import sysconfig

    import torch
    from torch.utils import cpp_extension

    includes = cpp_extension.include_paths("cuda") + [sysconfig.get_paths()["include"]]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_lib = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "lib64")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-DTORCH_EXTENSION_NAME=_C",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           *[f"-I{p}" for p in includes], TORCH_SRC, "-o", TORCH_EXT,
           f"-L{HERE}", "-lkm_b200", f"-L{torch_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
           "-ltorch_python", f"-L{cuda_lib}", "-lcudart", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("build of the PyTorch extension kernel_matmul_b200/_C.so failed")
    return TORCH_EXT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    if "--torch" in sys.argv:
        print(build_torch_extension(force="--force" in sys.argv))
