"""Compile the reference's own CUDA kernels for sm_100a into oracle/_ref/libref_wkv6_cuda.so.

Test / benchmark infrastructure only: the product never loads this library.  The source is the reference's
rwkv_kernel/jax_kernel/rwkv_kernels.cu, compiled where it lies in the reference tree (the directory ``WKV6_REFERENCE_DIR`` names)
with the reference's own flags (jax_rwkv_kernel.py:472-474: -O3 -DNDEBUG --expt-relaxed-constexpr,
hidden visibility, -D_N_ / -D_T_) except for the target architecture, plus the shim oracle/ref_cuda_shim.cu that gives
its three handlers C names.  _N_ = 64 and _T_ = 4096 fix the head size and the longest sequence, as in the reference.
Where the reference tree is absent (a GPU box) the prebuilt library is used as it is; build() then returns None when
there is none.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT_DIR, "libref_wkv6_cuda.so")
HEAD_SIZE, MAX_T = 64, 4096


def build(force: bool = False):
    ref = os.environ.get("WKV6_REFERENCE_DIR", "/root/reference")
    src = os.path.join(ref, "rwkv_kernel", "jax_kernel", "rwkv_kernels.cu")
    if not os.path.exists(src):
        return LIB if os.path.exists(LIB) else None
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(src):
        return LIB
    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-DNDEBUG", "--expt-relaxed-constexpr", "-std=c++17",
           "-Xcompiler", "-O3", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-w",
           f"-D_N_={HEAD_SIZE}", f"-D_T_={MAX_T}", "-I", os.path.dirname(src), "-shared", "-o", LIB,
           src, os.path.join(HERE, "ref_cuda_shim.cu"), "-lcudart"]
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
