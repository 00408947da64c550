"""Build oracle/_ref/: the reference's own CUDA kernels as shared libraries (test infrastructure).

The reference's kernel files depend only on the CUDA runtime, so they compile from where
they lie with a single nvcc command each (its JIT build through torch is not used). Nothing
is copied: nvcc reads the sources from the reference checkout and only the .so files are
written, into oracle/_ref/ (git-ignored). When the reference checkout is absent (for example
on a GPU machine that received prebuilt files) this is a no-op.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def build_ref(reference="/root/reference", verbose=False):
    src_dir = os.path.join(reference, "na1d_tensorcore")
    if not os.path.isdir(src_dir):
        return []
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    os.makedirs(OUT, exist_ok=True)
    built = []
    for dt, macro in (("bf16", "REF_BF16"), ("fp16", "REF_FP16")):
        so = os.path.join(OUT, f"libref_ana1d_{dt}.so")
        srcs = [os.path.join(HERE, "ref_cuda_shim.cu"), os.path.join(src_dir, f"{dt}_ana1d_kernel.cu")]
        if os.path.exists(so) and all(os.path.getmtime(so) > os.path.getmtime(s) for s in srcs):
            built.append(so)
            continue
        cmd = [nvcc, "-O3", "-shared", "-Xcompiler", "-fPIC", "-w",
               "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
               f"-D{macro}", f"-I{src_dir}", "-o", so] + srcs
        if verbose:
            print(" ".join(cmd))
        subprocess.check_call(cmd)
        built.append(so)
    return built


if __name__ == "__main__":
    print(build_ref(*(sys.argv[1:2]), verbose=True))
