#!/usr/bin/env python3
"""Builds the unmodified reference (its C core with the CUDA backend) as a shared library
under baseline/_ref, with the compiler flags of its own Makefile (CFLAGS, NVCCFLAGS and the
cuda-generic target's -gencode list, to which the B200's own architecture is added through
the Makefile's CUDA_GENERIC_ARCH_FLAGS variable so that nothing is compiled at load time).

    python baseline/build_reference.py /path/to/Kipp

The sources are copied, not changed.  bench.py --impl reference loads the library with
ctypes and drives it through its public API (src/kipp.h).
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
ARCH = ["-gencode", "arch=compute_80,code=sm_80", "-gencode", "arch=compute_90,code=sm_90",
        "-gencode", "arch=compute_100,code=sm_100", "-gencode", "arch=compute_80,code=compute_80"]


def run(cmd, cwd):
    print(" ".join(cmd), flush=True)
    subprocess.check_call(cmd, cwd=cwd)


def main() -> int:
    source = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("KIPP_REFERENCE_SOURCE", "")
    if not os.path.isdir(source):
        print("usage: build_reference.py /path/to/Kipp (or KIPP_REFERENCE_SOURCE)", file=sys.stderr)
        return 2
    src = os.path.join(REF, "src_tree")
    if os.path.isdir(src):
        shutil.rmtree(src)
    os.makedirs(REF, exist_ok=True)
    shutil.copytree(source, src, ignore=shutil.ignore_patterns(".git", "bench", "docs", "examples"))
    build = os.path.join(REF, "build")
    os.makedirs(build, exist_ok=True)
    cflags = ["-std=c11", "-O2", "-Wall", "-Wextra", "-Wpedantic", "-Werror", "-fPIC", "-Isrc"]
    nvccflags = ["-std=c++17", "-O2", "-I./src", "-I./cuda", "-Xcompiler=-Wall,-Wextra,-Werror,-fPIC"] + ARCH
    run(["gcc"] + cflags + ["-DKIPP_ENABLE_CUDA", "-c", "src/kipp.c", "-o", os.path.join(build, "kipp_cuda_core.o")], src)
    run(["gcc"] + cflags + ["-c", "src/kipp_kv_pool.c", "-o", os.path.join(build, "kipp_kv_pool.o")], src)
    run(["nvcc"] + nvccflags + ["-c", "src/cuda/kipp_cuda.cu", "-o", os.path.join(build, "kipp_cuda_bridge.o")], src)
    run(["nvcc"] + nvccflags + ["-c", "cuda/kipp_kernels.cu", "-o", os.path.join(build, "kipp_cuda_kernels.o")], src)
    run(["nvcc", "-shared"] + ARCH + [os.path.join(build, n) for n in
                                     ("kipp_cuda_core.o", "kipp_kv_pool.o", "kipp_cuda_bridge.o",
                                      "kipp_cuda_kernels.o")] + ["-lm", "-o", os.path.join(REF, "libkipp_ref.so")], src)
    print("built", os.path.join(REF, "libkipp_ref.so"))
    return 0


if __name__ == "__main__":
    sys.exit(main())
