"""CPU tier: the C-ABI library loads, exports every symbol the header declares, and validates
arguments without touching a GPU."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    from star_rwkv6_b200 import _lib
    return _lib


def test_header_symbols_exported(L):
    hdr = open(os.path.join(ROOT, "include", "wkv6_b200.h")).read()
    declared = set(re.findall(r"WKV6_API\s+[\w\s\*]+?\b(wkv6_\w+)\s*\(", hdr))
    assert declared, "no declarations found"
    assert declared == set(L.SYMBOLS)
    for name in declared:
        assert getattr(L.lib, name) is not None


def test_version(L):
    assert b"sm_100a" in L.lib.wkv6_version()


def _problem(L, **kw):
    p = L.Problem()
    p.B, p.T, p.H, p.N = 2, 8, 2, 64
    p.x_dtype = p.y_dtype = p.u_dtype = p.gu_dtype = p.s_dtype = L.F32
    for k, v in kw.items():
        setattr(p, k, v)
    return p


def test_validation_errors(L):
    lib = L.lib
    assert lib.wkv6_resolve_variant(ctypes.byref(_problem(L))) == L.VARIANT_SEQ
    assert lib.wkv6_resolve_variant(ctypes.byref(_problem(L, N=24))) == -2
    assert b"head size" in lib.wkv6_last_error()
    assert lib.wkv6_resolve_variant(ctypes.byref(_problem(L, x_dtype=L.F32, y_dtype=L.BF16))) == -2
    assert lib.wkv6_resolve_variant(ctypes.byref(_problem(L, row_stride=64))) == -1   # < H*N
    assert lib.wkv6_resolve_variant(ctypes.byref(_problem(L, row_stride=132))) == -1  # not a multiple of 8
    assert lib.wkv6_resolve_variant(ctypes.byref(_problem(L, variant=9))) == -1
    # null pointers are rejected before any launch
    p = _problem(L)
    assert lib.wkv6_forward(ctypes.byref(p), None, None, None, None, None, None, None, None, 0, None, None, None) == -1
    assert b"NULL" in lib.wkv6_last_error()


def test_workspace_queries(L):
    lib = L.lib
    p = _problem(L)
    assert lib.wkv6_backward_workspace_bytes(ctypes.byref(p), 0) == 0          # fp32 dense: staged in gw
    p = _problem(L, x_dtype=L.BF16, y_dtype=L.BF16, variant=L.VARIANT_SEQ)
    assert lib.wkv6_backward_workspace_bytes(ctypes.byref(p), 0) == 2 * 8 * 128 * 4
    assert lib.wkv6_ckpt_bytes(ctypes.byref(p)) == 0


def test_operator_rejects_cpu_tensors():
    import torch
    from star_rwkv6_b200.rwkv_kernel import RWKVKernelOperator
    op = RWKVKernelOperator(64, 16)
    z = torch.zeros(1, 4, 64)
    with pytest.raises(AssertionError):
        op(z, z, z, z, torch.zeros(1, 64))


def test_stage_and_copy_argument_checks(L):
    """Calls that must be refused before anything is launched (fake, never dereferenced addresses)."""
    lib = L.lib
    a = 0x1000                                                # an aligned, non-NULL address
    assert lib.wkv6_decode_ln_shift_mix(2, 7, L.BF16, 1e-5, a, a, a, a, a, None, None, None, a, None, None) == -2   # D odd
    assert lib.wkv6_decode_ln_shift_mix(2, 16384, L.BF16, 1e-5, a, a, a, a, a, None, None, None, a, None, None) == -2
    assert lib.wkv6_decode_ln_shift_mix(2, 64, L.BF16, 1e-5, a, a, a, None, a, None, None, None, a, None, None) == -1  # prev NULL
    assert lib.wkv6_decode_ln_shift_mix(2, 64, L.BF16, 1e-5, a + 2, a, a, a, a, None, None, None, a, None, None) == -1
    assert b"aligned" in lib.wkv6_last_error()
    assert lib.wkv6_decode_ln_shift_mix(2, 64, L.BF16, 1e-5, a, a, a, a, a, None, None, None, a, a, None) == -1     # mix1 without mu1
    assert lib.wkv6_decode_ln_shift_mix(2, 64, 77, 1e-5, a, a, a, a, a, None, None, None, a, None, None) == -1      # dtype
    assert lib.wkv6_decode_ln_shift_mix(0, 64, L.BF16, 1e-5, None, None, None, None, None, None, None, None, None, None, None) == 0
    bad = (ctypes.c_int32 * 5)(0, 1, 2, 2, 4)
    assert lib.wkv6_decode_lora_mix(2, 64, 8, L.BF16, a, a, a, a, a, a, bad, None) == -1
    assert b"permutation" in lib.wkv6_last_error()
    assert lib.wkv6_decode_lora_mix(2, 63, 8, L.BF16, a, a, a, a, a, a, None, None) == -2
    assert lib.wkv6_decode_lora_mix(2, 64, 8, L.F32, a, a + 4, a, a, a, a, None, None) == -1
    assert lib.wkv6_decode_relu_sq(-1, L.BF16, a, a, None) == -1
    assert lib.wkv6_decode_relu_sq(0, L.BF16, None, None, None) == 0
    assert lib.wkv6_decode_sigmoid_mul_add(5, L.BF16, a, None, a, a, None) == -1
    assert lib.wkv6_copy_2d_async(a, 8, a, 16, 16, 4, 0, None) == -1            # destination pitch below the width
    assert lib.wkv6_copy_2d_async(None, 16, a, 16, 16, 4, 0, None) == -1
    assert lib.wkv6_copy_2d_async(None, 0, None, 0, 0, 0, 0, None) == 0          # nothing to copy
    # the row sum and the scan-only summaries of the sequence-splitting path
    assert lib.wkv6_sum_rows(a, -1, 64, a, None) == -1
    assert lib.wkv6_sum_rows(None, 3, 64, a, None) == -1
    assert lib.wkv6_sum_rows(a, 3, 64, None, None) == -1
    assert lib.wkv6_sum_rows(None, 0, 0, None, None) == 0                        # nothing to sum
    pb = _problem(L, B=6, T=128, x_dtype=L.BF16, y_dtype=L.BF16)
    assert lib.wkv6_segment_summary_for_scan(ctypes.byref(pb), a, a, a, 0, 4, a, a, None) == -1   # 6 rows are not 4 segments each
    assert b"multiple" in lib.wkv6_last_error()
    assert lib.wkv6_segment_summary_for_scan(ctypes.byref(pb), a, a, a, 0, 0, a, a, None) == -1
    assert lib.wkv6_segment_summary_for_scan(ctypes.byref(pb), None, a, a, 0, 3, a, a, None) == -1
    pf = _problem(L, B=6, T=128)                                                 # fp32: no chunked variant
    assert lib.wkv6_segment_summary_for_scan(ctypes.byref(pf), a, a, a, 0, 3, a, a, None) == -2


def test_missing_library_fails_loudly():
    """Without the built CUDA library the package does not import: there is no CPU or framework fallback."""
    import subprocess
    import sys
    env = dict(os.environ, WKV6_B200_LIB="/nonexistent/libwkv6_b200.so")
    r = subprocess.run([sys.executable, "-c", "import star_rwkv6_b200"], cwd=ROOT, env=env, capture_output=True, text=True)
    assert r.returncode != 0 and "no fallback" in r.stderr


def test_product_never_touches_the_oracle():
    """The oracle is test infrastructure: no file of the package may import or load anything under oracle/."""
    pkg = os.path.join(ROOT, "star_rwkv6_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f), errors="ignore").read()
                assert not re.search(r"^\s*(from|import)\s+oracle\b", text, re.M), f
                assert "libwkv6_oracle" not in text and "oracle/" not in text, f
