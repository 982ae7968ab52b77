"""In-tree build of the native libraries (nvcc cross-compiles sm_100a without a GPU).

    libfluidml_b200_kernels.so   the CUDA kernel library behind include/fluidml_cuda.h
    libfluidml_b200.so           the C++ host (parser, converter, planners, executor) behind
                                 include/worker/executor.h and include/fluidml_executor.h

Run ``python -m fluidml_b200.build`` or call ``build_all()``.  Objects are rebuilt only when
their sources (or any header) are newer.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "fluidml_b200")
CSRC = os.path.join(PKG, "csrc")
LIBDIR = os.path.join(PKG, "lib")
OBJDIR = os.path.join(ROOT, "build", "obj")
INCLUDE = os.path.join(ROOT, "include")
# The toolchain is named explicitly: a CXX inherited from the environment may point at a
# wrapper that links libstdc++ statically, which breaks inside a Python process.
NVCC = os.environ.get("FLUIDML_NVCC", "/usr/local/cuda/bin/nvcc")
CXX = os.environ.get("FLUIDML_CXX", "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++")

KERNELS_SO = os.path.join(LIBDIR, "libfluidml_b200_kernels.so")
HOST_SO = os.path.join(LIBDIR, "libfluidml_b200.so")

NVCC_FLAGS = ["-ccbin", CXX, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-I", INCLUDE, "-I", os.path.join(CSRC, "kernels"),
              *os.environ.get("FLUIDML_NVCC_EXTRA", "").split()]  # e.g. -DFML_KERNEL_TRACE for a debug build
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-I", INCLUDE, "-I", os.path.join(CSRC, "host"),
             "-I", "/usr/local/cuda/include"]


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("build step failed: " + " ".join(cmd))
    if verbose and r.stdout.strip():
        print(r.stdout)
    return r.stdout


def build_kernels(verbose: bool = False, ptxas_info: bool = False) -> str:
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(OBJDIR, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "kernels", "*.cu")))
    hdrs = glob.glob(os.path.join(CSRC, "kernels", "*.cuh")) + glob.glob(os.path.join(INCLUDE, "*.h"))
    objs, jobs = [], []
    for s in srcs:
        o = os.path.join(OBJDIR, os.path.basename(s) + ".o")
        objs.append(o)
        if _newer(o, [s, *hdrs]):
            extra = ["-Xptxas", "-v"] if ptxas_info else []
            jobs.append([NVCC, *NVCC_FLAGS, *extra, "-c", s, "-o", o])
    with ThreadPoolExecutor(max_workers=8) as ex:
        outs = list(ex.map(lambda c: _run(c, verbose), jobs))
    if ptxas_info:
        for c, o in zip(jobs, outs):
            print(o)
    if jobs or _newer(KERNELS_SO, objs):
        _run([NVCC, "-shared", "-o", KERNELS_SO, *objs, "-gencode",
              "arch=compute_100a,code=sm_100a"], verbose)
    return KERNELS_SO


def build_cli(verbose: bool = False) -> str:
    """fluidml-compiler, the counterpart of the reference's bin/compiler."""
    bindir = os.path.join(PKG, "bin")
    os.makedirs(bindir, exist_ok=True)
    src = os.path.join(CSRC, "cli", "compiler.cpp")
    exe = os.path.join(bindir, "fluidml-compiler")
    if _newer(exe, [src, HOST_SO, KERNELS_SO]):
        _run([CXX, *CXX_FLAGS, src, "-o", exe, "-L", LIBDIR, "-lfluidml_b200", "-lfluidml_b200_kernels",
              "-Wl,-rpath,$ORIGIN/../lib"], verbose)
    return exe


def build_host(verbose: bool = False) -> str:
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(OBJDIR, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "host", "*.cpp")))
    if not srcs:
        return ""
    hdrs = glob.glob(os.path.join(CSRC, "host", "*.h")) + \
        glob.glob(os.path.join(INCLUDE, "**", "*.h"), recursive=True)
    objs, jobs = [], []
    for s in srcs:
        o = os.path.join(OBJDIR, "host_" + os.path.basename(s) + ".o")
        objs.append(o)
        if _newer(o, [s, *hdrs]):
            jobs.append([CXX, *CXX_FLAGS, "-c", s, "-o", o])
    with ThreadPoolExecutor(max_workers=8) as ex:
        list(ex.map(lambda c: _run(c, verbose), jobs))
    if jobs or _newer(HOST_SO, [*objs, KERNELS_SO]):
        _run([CXX, "-shared", "-o", HOST_SO, *objs, "-L", LIBDIR, "-lfluidml_b200_kernels",
              "-Wl,-rpath,$ORIGIN"], verbose)
    return HOST_SO


def build_all(verbose: bool = False) -> None:
    build_kernels(verbose)
    build_host(verbose)
    build_cli(verbose)


if __name__ == "__main__":
    build_all(verbose="-v" in sys.argv)
    print("built", KERNELS_SO, HOST_SO if os.path.exists(HOST_SO) else "")
