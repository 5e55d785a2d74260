"""The typed XLA FFI source (csrc/wkv6_xla_ffi.cc) is only compiled where jaxlib's headers exist, which is not here.  This
test type-checks it against a compile-only stand-in for ``xla/ffi/api/ffi.h`` (tests/fake_xla_ffi): what it verifies is the
file's own consistency and, above all, that its calls into this library match ``include/wkv6_b200.h`` (argument counts and
types of wkv6_forward / wkv6_backward / the size queries).  It says nothing about the real header."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_ffi_source_type_checks(tmp_path):
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    if not os.path.exists(nvcc) and shutil.which("nvcc") is None:
        pytest.skip("no nvcc")
    src = os.path.join(ROOT, "star_rwkv6_b200", "csrc", "wkv6_xla_ffi.cc")
    inc = os.path.join(ROOT, "tests", "fake_xla_ffi")
    cmd = [nvcc if os.path.exists(nvcc) else "nvcc", "-x", "cu", "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17",
           "-Xcompiler", "-fPIC,-Wall", "-I", inc, "-c", src, "-o", str(tmp_path / "ffi.o")]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-3000:]
    # the three handler symbols the Python side registers are defined
    nm = subprocess.run(["nm", "-g", str(tmp_path / "ffi.o")], capture_output=True, text=True).stdout
    for sym in ("wkv6_ffi_forward", "wkv6_ffi_backward", "wkv6_ffi_forward_with_state"):
        assert f" T {sym}" in nm, sym
