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
