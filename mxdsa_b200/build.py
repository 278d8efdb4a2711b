"""In-tree build of the native parts (run as ``python -m mxdsa_b200.build``).

  lib/libmxdsa.so   the C ABI + all CUDA kernels, compiled for sm_100a only
  lib/mxdsa_ext*.so the PyTorch extension module (C++ binding over the C ABI)

Both are written next to the sources so that they travel with the tree; nothing is installed
into site-packages and nothing is JIT-cached elsewhere.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "lib")
NVCC = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "--use_fast_math", "-Xcompiler", "-fPIC"]


def _newer(target: str, sources) -> bool:
    if not os.path.isfile(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _sources(*ext):
    out = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith(ext)]
    out.append(os.path.join(HERE, "..", "include", "mxdsa.h"))
    return out


def build_lib(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIB, exist_ok=True)
    target = os.path.join(LIB, "libmxdsa.so")
    if force or _newer(target, _sources(".cu", ".cuh", ".h")):
        # the attention kernels use fast-math intrinsics on purpose; the pack and selection kernels need IEEE arithmetic
        objs = []
        ieee = [f for f in NVCC_FLAGS if f != "--use_fast_math"]
        for name, flags in (("mxdsa_lib.cu", NVCC_FLAGS), ("pack_kernels.cu", ieee), ("topk_kernels.cu", ieee)):
            obj = os.path.join(LIB, name.replace(".cu", ".o"))
            cmd = [NVCC, *flags, "-c", "-o", obj, os.path.join(CSRC, name)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            subprocess.run(cmd, check=True)
            objs.append(obj)
        subprocess.run([NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", target, *objs, "-lcudart"],
                       check=True)
        for obj in objs:
            os.remove(obj)
    return target


def build_ext(force: bool = False) -> str:
    """The torch extension: plain C++ (no CUDA code), links libmxdsa.so through an $ORIGIN rpath."""
    import torch
    os.makedirs(LIB, exist_ok=True)
    target = os.path.join(LIB, "mxdsa_ext.so")
    src = os.path.join(CSRC, "torch_binding.cpp")
    if force or _newer(target, [src, os.path.join(HERE, "..", "include", "mxdsa.h")]):
        troot = os.path.dirname(torch.__file__)
        cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
        cmd = ["c++", "-O2", "-std=c++17", "-fPIC", "-shared", "-DNDEBUG", "-D_GLIBCXX_USE_CXX11_ABI=1",
               f"-I{os.path.join(HERE, '..', 'include')}", f"-I{cuda_inc}",
               f"-I{os.path.join(troot, 'include')}",
               f"-I{os.path.join(troot, 'include', 'torch', 'csrc', 'api', 'include')}",
               f"-I{sysconfig.get_path('include')}", src, "-o", target,
               f"-L{LIB}", "-lmxdsa", "-Wl,-rpath,$ORIGIN",
               f"-L{os.path.join(troot, 'lib')}", f"-Wl,-rpath,{os.path.join(troot, 'lib')}",
               "-ltorch_python", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda"]
        subprocess.run(cmd, check=True)
    return target


def build_all(force: bool = False) -> None:
    build_lib(force)
    build_ext(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print("built", os.listdir(LIB))
