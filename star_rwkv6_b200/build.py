"""Build the CUDA library in-tree: star_rwkv6_b200/libwkv6_b200.so (sm_100a only).

``python star_rwkv6_b200/build.py`` (run as a script, so that it works before the library exists) compiles every ``.cu`` under ``csrc/`` with nvcc and links
one shared object that exports the C ABI declared in ``include/wkv6_b200.h``.  nvcc
cross-compiles, so no GPU is needed to build.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libwkv6_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def xla_ffi_include_dir():
    """Directory of jaxlib's xla/ffi/api/ffi.h, or None: the typed-FFI handlers (csrc/wkv6_xla_ffi.cc) are compiled
    into the library only where JAX is installed."""
    try:
        import jax.ffi
        inc = jax.ffi.include_dir()
    except Exception:
        return None
    return inc if os.path.exists(os.path.join(inc, "xla", "ffi", "api", "ffi.h")) else None


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = glob.glob(os.path.join(CSRC, "*")) + glob.glob(os.path.join(PKG, "..", "include", "*.h"))
    return any(os.path.getmtime(f) > t for f in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    objs = []
    procs = []
    for src in sources():
        obj = os.path.splitext(src)[0] + ".o"
        cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
        procs.append((cmd, subprocess.Popen(cmd)))
        objs.append(obj)
    inc = xla_ffi_include_dir()
    if inc is not None:   # exported with default visibility: the handler symbols are what jax.ffi.pycapsule looks up
        src, obj = os.path.join(CSRC, "wkv6_xla_ffi.cc"), os.path.join(CSRC, "wkv6_xla_ffi.o")
        flags = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC"]
        cmd = [nvcc, "-x", "cu"] + flags + ["-I", inc, "-c", src, "-o", obj]
        procs.append((cmd, subprocess.Popen(cmd)))
        objs.append(obj)
    for cmd, pr in procs:
        if pr.wait() != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
    subprocess.check_call([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIB] + objs + ["-lcudart"])
    return LIB


def build_variant(out_path: str, extra_flags) -> str:
    """The same library compiled with extra nvcc flags (e.g. ``-DWKV6_TIMING``: phase stamps inside the chunked kernels and
    the exports that read them) into ``out_path``; objects go to a temporary directory, the in-tree library is untouched.
    ``WKV6_B200_LIB=<out_path>`` makes the package load it."""
    import tempfile
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    with tempfile.TemporaryDirectory() as tmp:
        procs, objs = [], []
        for src in sources():
            obj = os.path.join(tmp, os.path.splitext(os.path.basename(src))[0] + ".o")
            cmd = [nvcc] + NVCC_FLAGS + list(extra_flags) + ["-c", src, "-o", obj]
            procs.append((cmd, subprocess.Popen(cmd)))
            objs.append(obj)
        for cmd, pr in procs:
            if pr.wait() != 0:
                raise RuntimeError("nvcc failed: " + " ".join(cmd))
        subprocess.check_call([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", out_path] + objs + ["-lcudart"])
    return out_path


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
