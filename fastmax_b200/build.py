"""Builds the native parts of fastmax_b200 in-tree for sm_100a.

``python -m fastmax_b200.build`` compiles

* ``fastmax_b200/libfastmax_b200.so`` -- the CUDA kernels and the C ABI declared
  in ``include/fastmax_b200.h`` (plain nvcc, no torch dependency), and
* ``fastmax_cuda*.so`` -- the torch C++ extension that exposes the reference's
  ``forwardpass`` / ``backwardpass`` entry points on top of that C ABI
  (only with ``--torch-ext``; it needs the torch headers and takes a minute).

nvcc cross-compiles without a GPU, so the build runs anywhere the CUDA toolkit
is installed.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libfastmax_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-I" + os.path.join(ROOT, "include"), "-I" + CSRC,
]


def _newer(target: str, sources) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile every ``csrc/*.cu`` into the shared library; returns its path."""
    cus = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    deps = cus + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    if not force and _newer(LIB, deps):
        return LIB
    objs = []
    procs = []
    os.makedirs(os.path.join(PKG, "build"), exist_ok=True)
    for cu in cus:
        obj = os.path.join(PKG, "build", os.path.basename(cu)[:-3] + ".o")
        objs.append(obj)
        if not force and _newer(obj, [cu] + deps[len(cus):]):
            continue
        cmd = ["nvcc"] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", cu, "-o", obj]
        procs.append((cu, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for cu, pr in procs:
        out, _ = pr.communicate()
        if verbose or pr.returncode:
            sys.stderr.write(out)
        if pr.returncode:
            raise RuntimeError(f"nvcc failed on {cu}")
    subprocess.check_call(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIB]
                          + objs + ["-lcudart", "-lcuda"])
    return LIB


def build_torch_extension(force: bool = False) -> str:
    """Compile the ``fastmax_cuda`` torch extension next to the package."""
    import sysconfig

    import torch
    from torch.utils import cpp_extension

    build_library()
    src = os.path.join(CSRC, "torch_binding.cpp")
    suffix = sysconfig.get_config_var("EXT_SUFFIX")
    target = os.path.join(ROOT, "fastmax_cuda" + suffix)
    if not force and _newer(target, [src, os.path.join(ROOT, "include", "fastmax_b200.h")]):
        return target
    inc = cpp_extension.include_paths("cuda")
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=fastmax_cuda",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           "-I" + os.path.join(ROOT, "include"), "-I" + sysconfig.get_paths()["include"]]
    cmd += ["-I" + p for p in inc]
    cmd += [src, "-o", target, "-L" + tlib, "-L" + PKG, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda",
            "-ltorch", "-ltorch_python", "-l:libfastmax_b200.so", "-L/usr/local/cuda/lib64", "-lcudart",
            "-Wl,-rpath,$ORIGIN/fastmax_b200", "-Wl,-rpath," + tlib]
    subprocess.check_call(cmd)
    return target


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_library(force=force, verbose="-v" in sys.argv))
    if "--torch-ext" in sys.argv:
        print(build_torch_extension(force=force))
