"""In-tree build of the native libraries (nvcc / g++ called directly, no build system).

``libkuiper_b200.so``  - the sm_100a kernels behind the C ABI of ``include/kuiper_b200.h``
``libkuiper_llama.so`` - the C++ host side (base / tensor / op / model) on top of it

Both land in ``mykuiperllama_b200/lib/`` so that they travel with the source tree.
"""
from __future__ import annotations

import glob
import hashlib
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
OBJ_DIR = os.path.join(PKG, "lib", "obj")

# KUIPER_TRACE=1 in the environment selects a second kernel library built with -DKUIPER_TRACE (per-CTA clock
# readings inside the kernels, read back with kuiper_*_trace_read); the shipped library has none of it
TRACE = os.environ.get("KUIPER_TRACE", "0") == "1"
KERNEL_LIB = os.path.join(LIB_DIR, "libkuiper_b200_trace.so" if TRACE else "libkuiper_b200.so")
HOST_LIB = os.path.join(LIB_DIR, "libkuiper_llama.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA extension cannot be built")


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if verbose and res.stdout:
        print(res.stdout, flush=True)
    if res.returncode != 0:
        raise RuntimeError(f"build step failed ({res.returncode}): {' '.join(cmd)}\n{res.stdout}")


def build_kernels(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "kernels", "*.cu")))
    hdrs = sorted(glob.glob(os.path.join(CSRC, "kernels", "*.cuh"))) + [os.path.join(ROOT, "include", "kuiper_b200.h")]
    objs = []
    flags = NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + (["-DKUIPER_TRACE=1"] if TRACE else [])
    for src in srcs:
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ("_trace.o" if TRACE else ".o"))
        objs.append(obj)
        if force or ptxas_info or _stale(obj, [src] + hdrs):
            _run([_nvcc(), *flags, "-I", os.path.join(ROOT, "include"), "-I", os.path.join(CSRC, "kernels"),
                  "-c", src, "-o", obj], verbose or ptxas_info)
    if force or _stale(KERNEL_LIB, objs):
        _run([_nvcc(), "-shared", "-o", KERNEL_LIB, *objs, "-cudart", "shared"], verbose)
    return KERNEL_LIB


def _cuda_home() -> str:
    return os.path.dirname(os.path.dirname(_nvcc()))


def build_host(force: bool = False, verbose: bool = False) -> str | None:
    """C++ host side; skipped while the sources are absent."""
    src_dir = os.path.join(CSRC, "kuiper", "source")
    srcs = sorted(glob.glob(os.path.join(src_dir, "**", "*.cpp"), recursive=True))
    if not srcs:
        return None
    inc = os.path.join(CSRC, "kuiper", "include")
    hdrs = sorted(glob.glob(os.path.join(inc, "**", "*.h"), recursive=True)) + \
        sorted(glob.glob(os.path.join(src_dir, "**", "*.h"), recursive=True)) + \
        [os.path.join(ROOT, "include", "kuiper_b200.h"), os.path.join(ROOT, "include", "kuiper_llama.h")]
    hdrs = [h for h in hdrs if os.path.exists(h)]
    os.makedirs(OBJ_DIR, exist_ok=True)
    objs = []
    cuda = _cuda_home()
    for src in srcs:
        tag = hashlib.md5(os.path.relpath(src, src_dir).encode()).hexdigest()[:8]
        obj = os.path.join(OBJ_DIR, f"host_{os.path.basename(src)[:-4]}_{tag}.o")
        objs.append(obj)
        if force or _stale(obj, [src] + hdrs):
            _run(["g++", "-O2", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-parameter",
                  "-I", inc, "-I", src_dir, "-I", os.path.join(ROOT, "include"), "-I", os.path.join(cuda, "include"),
                  "-c", src, "-o", obj], verbose)
    if force or _stale(HOST_LIB, objs + [KERNEL_LIB]):
        _run(["g++", "-shared", "-o", HOST_LIB, *objs, "-L", LIB_DIR, "-lkuiper_b200",
              "-L", os.path.join(cuda, "lib64"), "-lcudart", "-Wl,-rpath,$ORIGIN", "-ldl", "-lpthread"], verbose)
    return HOST_LIB


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_kernels(force=force, verbose=verbose)
    build_host(force=force, verbose=verbose)


if __name__ == "__main__":
    build_kernels(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv)
    build_host(force="--force" in sys.argv, verbose=True)
