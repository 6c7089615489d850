"""In-tree build of libmps_b200.so and the MergePathSpMM command-line program (nvcc, sm_100a only)."""
from __future__ import annotations

import os
import shutil
import subprocess

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIBDIR = os.path.join(PKG, "lib")
LIB = os.path.join(LIBDIR, "libmps_b200.so")
CLI = os.path.join(LIBDIR, "MergePathSpMM")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-I" + os.path.join(ROOT, "include"), "-I" + CSRC] + os.environ.get("MPS_EXTRA_NVCC_FLAGS", "").split()


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libmps_b200.so cannot be built")
    return exe


def _newer(target: str, sources) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _sources(names):
    return [os.path.join(CSRC, n) for n in names]


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compiles every source to an object (in parallel) and links libmps_b200.so."""
    from concurrent.futures import ThreadPoolExecutor
    srcs = _sources(["mps_api.cu", "mps_spmm_f32.cu", "mps_spmm_f32_scaled.cu", "mps_spmm_f16.cu", "mps_noalloc.cu", "mps_multi.cu", "mps_probe.cu", "convert_device.cu", "csr_io.cpp", "convert.cpp", "host_check.cpp", "partition_host.cpp"])
    deps = srcs + _sources(["mps_kernels.cuh", "mps_dispatch.cuh", "mps_internal.h", "mps_plan.h"]) + [os.path.join(ROOT, "include", "mps.h")]
    if not force and _newer(LIB, deps):
        return LIB
    os.makedirs(LIBDIR, exist_ok=True)
    objdir = os.path.join(PKG, "build")
    os.makedirs(objdir, exist_ok=True)
    flags = ARCH + COMMON + ["-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-Xcompiler", "-pthread"]
    if verbose:
        flags = ["-Xptxas=-v"] + flags

    def compile_one(src):
        obj = os.path.join(objdir, os.path.basename(src) + ".o")
        subprocess.run([_nvcc()] + flags + ["-c", "-o", obj, src], check=True)
        return obj

    with ThreadPoolExecutor(max_workers=len(srcs)) as pool:
        objs = list(pool.map(compile_one, srcs))
    subprocess.run([_nvcc()] + ARCH + ["-shared", "-o", LIB] + objs + ["-ldl", "-lz"], check=True)
    return LIB


def build_cli(force: bool = False) -> str:
    """MergePathSpMM (the reference's entry point) and npz_to_csr (its converter script), linked to the library."""
    build_library(force)
    for exe, name in ((CLI, "bench_main.cpp"), (os.path.join(LIBDIR, "npz_to_csr"), "npz_to_csr_main.cpp")):
        src = os.path.join(CSRC, name)
        if not force and _newer(exe, [src, LIB]):
            continue
        cmd = [_nvcc()] + ARCH + COMMON + ["-Xcompiler", "-pthread", "-o", exe, src, "-L" + LIBDIR, "-lmps_b200",
                                          "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"]
        subprocess.run(cmd, check=True)
    twin = CLI + "_fp16"  # the reference's fp16 program has the same argv; the program looks at its own name
    if not os.path.exists(twin) or os.path.getmtime(twin) < os.path.getmtime(CLI):
        if os.path.lexists(twin):
            os.remove(twin)
        shutil.copy2(CLI, twin)
    return CLI


if __name__ == "__main__":
    print(build_library(force=True, verbose=False))
    print(build_cli(force=True))
