"""Ahead-of-time build of the CUDA library for sm_100a (in-tree, plain nvcc, no torch headers).

Every .cu under csrc/ is compiled to an object of its own (in parallel, only when it or a header changed) and the
objects are linked into libna1d_b200.so next to this file.
"""
import os
import shutil
import subprocess
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "libna1d_b200.so")

NVCC_FLAGS = ["-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo"]


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers():
    return [os.path.join(CSRC, f) for f in os.listdir(CSRC) if not f.endswith(".cu")] + [
        os.path.join(os.path.dirname(PKG), "include", "na1d_b200.h")]


def _deps():
    return sources() + _headers()


def is_stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(p) > t for p in _deps())


def build_library(force=False, verbose=False, extra_flags=()):
    """Compile every .cu under csrc/ and link libna1d_b200.so."""
    if not force and not is_stale():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot build libna1d_b200.so")
    os.makedirs(OBJ, exist_ok=True)
    newest_header = max(os.path.getmtime(p) for p in _headers())
    flags = NVCC_FLAGS + list(extra_flags)
    stamp = os.path.join(OBJ, "flags.txt")
    same_flags = os.path.exists(stamp) and open(stamp).read() == " ".join(flags)

    def compile_one(src):
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        if (not force and same_flags and os.path.exists(obj) and
                os.path.getmtime(obj) >= max(os.path.getmtime(src), newest_header)):
            return obj
        cmd = [nvcc] + flags + ["-c", "-o", obj, src]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, sources()))
    open(stamp, "w").write(" ".join(flags))
    cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB] + objs
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build_library(force=True, verbose=True))
