"""Builds the two artefacts of the package, in-tree:

* ``csrc/b200_contraction.cubin`` -- every kernel, compiled by nvcc for sm_100a only. This is
  the object a ``#hal.executable.object`` would carry.
* ``libiree_b200.so``             -- the host-side C ABI (``include/iree_b200.h``), compiled by
  g++. It opens libcuda / libnccl at run time, so it also loads on a machine without a GPU.

Run as ``python -m iree_b200.build``. Nothing here needs a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
CUBIN = os.path.join(CSRC, "b200_contraction.cubin")
LIB = os.path.join(HERE, "libiree_b200.so")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")

KERNEL_SOURCES = ["contraction_sm100.cu", "contraction_pair_sm100.cu", "w4a16_sm100.cu", "w4a16_wt_sm100.cu", "w4a16_decode_tc_sm100.cu",
                  "mmt4d_sm100.cu", "mmt4d_generic_sm100.cu", "data_tiling_sm100.cu", "tiling_tma_sm100.cu", "pack_vnni_sm100.cu"]
HOST_SOURCES = ["hal_b200.cc", "parameters.cc", "w4a16_noalloc.cu"]
HEADERS = ["sm100_ptx.cuh", "w4a16_decode.cuh", "w4a16_decode_tc.h", "hal_b200_internal.h", os.path.join("..", "..", "include", "iree_b200.h")]


def _newer(target: str, sources) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources if os.path.exists(s))


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    out = subprocess.run(cmd, capture_output=True, text=True)
    if out.returncode != 0:
        raise RuntimeError("build step failed: %s\n%s\n%s" % (" ".join(cmd), out.stdout, out.stderr))
    if verbose and (out.stdout or out.stderr):
        print(out.stdout + out.stderr, flush=True)


def build_cubin(force: bool = False, verbose: bool = False) -> str:
    srcs = [os.path.join(CSRC, s) for s in KERNEL_SOURCES if os.path.exists(os.path.join(CSRC, s))]
    deps = srcs + [os.path.join(CSRC, h) for h in HEADERS]
    if not force and _newer(CUBIN, deps):
        return CUBIN
    nvcc = shutil.which("nvcc") or os.path.join(CUDA_HOME, "bin", "nvcc")
    if not os.path.exists(nvcc):
        if os.path.exists(CUBIN):
            return CUBIN  # a prebuilt cubin travelled with the tree
        raise RuntimeError("nvcc not found and no prebuilt cubin at " + CUBIN)
    # One translation unit (the sources are #included by a tiny driver file) so that a single
    # cubin carries every export, as one hal.executable.object must.
    unit = os.path.join(CSRC, "_all_kernels.cu")
    with open(unit, "w") as f:
        for s in srcs:
            f.write('#include "%s"\n' % os.path.basename(s))
    try:
        _run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xptxas", "-v" if verbose else "-O3", "-cubin", "-o", CUBIN, unit], verbose)
    finally:
        os.remove(unit)
    return CUBIN


def build_host(force: bool = False, verbose: bool = False) -> str:
    srcs = [os.path.join(CSRC, s) for s in HOST_SOURCES]
    deps = srcs + [os.path.join(CSRC, h) for h in HEADERS]
    if not force and _newer(LIB, deps):
        return LIB
    nvcc = shutil.which("nvcc") or os.path.join(CUDA_HOME, "bin", "nvcc")
    if not os.path.exists(nvcc):
        if os.path.exists(LIB):
            return LIB
        raise RuntimeError("nvcc not found and no prebuilt " + LIB)
    # nvcc drives g++ for hal_b200.cc and compiles the one .cu that carries host code. The CUDA
    # runtime is linked statically; it opens the driver library lazily, so the result still
    # loads on a machine without a GPU.
    _run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O2", "-std=c++17", "-shared",
          "-cudart", "static", "-Xcompiler", "-fPIC,-Wall", "-o", LIB] + srcs + ["-ldl", "-lpthread"], verbose)
    return LIB


def build_all(force: bool = False, verbose: bool = False):
    return build_cubin(force, verbose), build_host(force, verbose)


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv, verbose=True))
