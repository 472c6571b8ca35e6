"""In-tree build of the native parts: libmxfp6.so (CUDA kernels + C ABI, sm_100a), the stand-alone C++ harness
matmul_host, and the
tk_kernel Python extension (pybind11, same module/function names as the reference's binding,
include/pyutils/pyutils.cuh:55-72 and kernels/gemm/bf16fp32/Makefile:41,51-52).

    python hipkittensp_b200/build.py            # build what is out of date
    python hipkittensp_b200/build.py --force

(run as a script: importing the package needs the library this builds)
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libmxfp6.so")
EXT = os.path.join(PKG, "tk_kernel" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
CUDA_HOME = os.path.dirname(os.path.dirname(NVCC))

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "-Xcompiler", "-fPIC", "-cudart", "shared", "-Xlinker", "-rpath,/usr/local/cuda/lib64"]


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _sources() -> list[str]:
    out = [os.path.join(ROOT, "include", "mxfp6.h")]
    for f in sorted(os.listdir(CSRC)):
        out.append(os.path.join(CSRC, f))
    return out


def build_lib(force: bool = False, verbose: bool = False) -> str:
    srcs = _sources()
    if not force and _newer(LIB, srcs):
        return LIB
    cmd = [NVCC, *NVCC_FLAGS, "-shared", "-Xptxas", "-v", "-o", LIB, os.path.join(CSRC, "mxfp6_api.cu")]
    res = subprocess.run(cmd, capture_output=True, text=True)
    with open(os.path.join(PKG, "ptxas_report.txt"), "w") as f:
        f.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stderr)
    return LIB


def build_ext(force: bool = False) -> str:
    import pybind11

    src = os.path.join(CSRC, "tk_kernel.cpp")
    if not force and _newer(EXT, [src, LIB, os.path.join(ROOT, "include", "mxfp6.h")]):
        return EXT
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden",
           "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], "-I", os.path.join(ROOT, "include"),
           "-I", os.path.join(CUDA_HOME, "include"), src, "-o", EXT, "-L", PKG, "-lmxfp6",
           "-L", os.path.join(CUDA_HOME, "lib64"), "-lcudart", "-Wl,-rpath,$ORIGIN"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("g++ failed:\n" + res.stdout + res.stderr)
    return EXT


HOST = os.path.join(PKG, "matmul_host")


def build_host(force: bool = False) -> str:
    """The stand-alone C++ harness over the C ABI (counterpart of the reference's `matmul_host` programs)."""
    src = os.path.join(CSRC, "matmul_host.cpp")
    if not force and _newer(HOST, [src, LIB, os.path.join(ROOT, "include", "mxfp6.h")]):
        return HOST
    cuda_lib = os.path.join(CUDA_HOME, "lib64")
    cmd = ["g++", "-O2", "-std=c++17", "-fopenmp", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(CUDA_HOME, "include"),
           src, "-o", HOST, "-L", PKG, "-lmxfp6", "-L", cuda_lib, "-lcudart", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + cuda_lib]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("g++ failed:\n" + res.stdout + res.stderr)
    return HOST


def build_all(force: bool = False, verbose: bool = False):
    return build_lib(force, verbose), build_ext(force), build_host(force)


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv, verbose=True))
