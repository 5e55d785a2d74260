"""ctypes binding of libwkv6_b200.so (the C ABI in include/wkv6_b200.h).

The library is required: there is no CPU or framework fallback.  If it has not been built,
importing this module raises with the build command.
"""
from __future__ import annotations

import ctypes
import os

PKG = os.path.dirname(os.path.abspath(__file__))
# WKV6_B200_LIB selects another build of the same library (e.g. one compiled with extra instrumentation)
LIB_PATH = os.environ.get("WKV6_B200_LIB") or os.path.join(PKG, "libwkv6_b200.so")

BF16, F16, F32 = 0, 1, 2
VARIANT_AUTO, VARIANT_SEQ, VARIANT_CHUNK = 0, 1, 2
VARIANTS = {"auto": VARIANT_AUTO, "seq": VARIANT_SEQ, "chunk": VARIANT_CHUNK}

# every symbol include/wkv6_b200.h declares
SYMBOLS = (
    "wkv6_last_error", "wkv6_version", "wkv6_device_status", "wkv6_debug_inject", "wkv6_resolve_variant", "wkv6_forward", "wkv6_ckpt_bytes",
    "wkv6_backward", "wkv6_backward_workspace_bytes", "wkv6_backward_static_scratch", "wkv6_static_scratch_bytes",
    "wkv6_decode", "wkv6_decode_gated", "wkv6_decode_ln_shift_mix", "wkv6_decode_lora_mix", "wkv6_decode_relu_sq",
    "wkv6_decode_sigmoid_mul_add", "wkv6_softmax_xent_bf16", "wkv6_segment_summary", "wkv6_segment_summary_for_scan", "wkv6_state_scan", "wkv6_backward_seeded", "wkv6_sum_rows",
    "wkv6_groupnorm_gate_forward", "wkv6_groupnorm_gate_backward", "wkv6_groupnorm_gate_workspace_bytes",
    "wkv6_groupnorm_silu_gate_forward", "wkv6_groupnorm_silu_gate_backward",
    "wkv6_shift_mix_forward", "wkv6_shift_mix_backward", "wkv6_shift_mix_workspace_bytes", "wkv6_copy_2d_async",
    "wkv6_relu_sq_forward", "wkv6_relu_sq_backward", "wkv6_sigmoid_mul_forward", "wkv6_sigmoid_mul_backward",
    "wkv6_xla_forward", "wkv6_xla_backward", "wkv6_xla_forward_with_state", "wkv6_xla_forward_ckpt", "wkv6_xla_backward_ws",
    "wkv6_xla_buffer_bytes", "wkv6_xla_descriptor", "wkv6_xla_target",
)


class Problem(ctypes.Structure):
    _fields_ = [
        ("B", ctypes.c_int32), ("T", ctypes.c_int32), ("H", ctypes.c_int32), ("N", ctypes.c_int32),
        ("x_dtype", ctypes.c_int32), ("y_dtype", ctypes.c_int32), ("u_dtype", ctypes.c_int32),
        ("gu_dtype", ctypes.c_int32), ("s_dtype", ctypes.c_int32), ("variant", ctypes.c_int32),
        ("row_stride", ctypes.c_int64), ("batch_stride", ctypes.c_int64),
    ]


class WKV6Error(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"wkv6_b200 error {code}: {msg}")
        self.code = code


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python star_rwkv6_b200/build.py` "
            "(nvcc, sm_100a). There is no fallback path.")
    lib = ctypes.CDLL(LIB_PATH)
    vp, i32, i64p, sz = ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p, ctypes.c_size_t
    pp = ctypes.POINTER(Problem)
    lib.wkv6_last_error.restype = ctypes.c_char_p
    lib.wkv6_last_error.argtypes = []
    lib.wkv6_version.restype = ctypes.c_char_p
    lib.wkv6_version.argtypes = []
    lib.wkv6_device_status.restype = ctypes.c_int
    lib.wkv6_device_status.argtypes = []
    lib.wkv6_debug_inject.restype = ctypes.c_int
    lib.wkv6_debug_inject.argtypes = [ctypes.c_int32, ctypes.c_int64]
    lib.wkv6_resolve_variant.restype = ctypes.c_int
    lib.wkv6_resolve_variant.argtypes = [pp]
    lib.wkv6_forward.restype = ctypes.c_int
    lib.wkv6_forward.argtypes = [pp, vp, vp, vp, vp, vp, vp, vp, i64p, i32, vp, vp, vp]
    lib.wkv6_ckpt_bytes.restype = sz
    lib.wkv6_ckpt_bytes.argtypes = [pp]
    lib.wkv6_backward.restype = ctypes.c_int
    lib.wkv6_backward.argtypes = [pp] + [vp] * 11 + [vp, vp, sz, vp]
    lib.wkv6_backward_workspace_bytes.restype = sz
    lib.wkv6_backward_workspace_bytes.argtypes = [pp, ctypes.c_int]
    lib.wkv6_backward_static_scratch.restype = ctypes.c_int
    lib.wkv6_backward_static_scratch.argtypes = [pp] + [vp] * 11 + [vp]
    lib.wkv6_static_scratch_bytes.restype = sz
    lib.wkv6_static_scratch_bytes.argtypes = []
    lib.wkv6_decode.restype = ctypes.c_int
    lib.wkv6_decode.argtypes = [pp, vp, vp, vp, vp, vp, vp, vp, i64p, i32, vp, vp]
    lib.wkv6_decode_gated.restype = ctypes.c_int
    lib.wkv6_decode_gated.argtypes = [pp, vp, vp, vp, vp, vp, vp, vp, vp, ctypes.c_float, vp, vp, i64p, i32, vp, vp]
    lib.wkv6_decode_ln_shift_mix.restype = ctypes.c_int
    lib.wkv6_decode_ln_shift_mix.argtypes = [i32, i32, i32, ctypes.c_float] + [vp] * 11
    lib.wkv6_decode_lora_mix.restype = ctypes.c_int
    lib.wkv6_decode_lora_mix.argtypes = [i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, ctypes.POINTER(ctypes.c_int32), vp]
    lib.wkv6_decode_relu_sq.restype = ctypes.c_int
    lib.wkv6_decode_relu_sq.argtypes = [ctypes.c_int64, i32, vp, vp, vp]
    lib.wkv6_decode_sigmoid_mul_add.restype = ctypes.c_int
    lib.wkv6_decode_sigmoid_mul_add.argtypes = [ctypes.c_int64, i32, vp, vp, vp, vp, vp]
    lib.wkv6_softmax_xent_bf16.restype = ctypes.c_int
    lib.wkv6_softmax_xent_bf16.argtypes = [ctypes.c_int64, i32, vp, i64p, ctypes.c_float, vp, vp]
    lib.wkv6_segment_summary.restype = ctypes.c_int
    lib.wkv6_segment_summary.argtypes = [pp, vp, vp, vp, ctypes.c_int, vp, vp, vp]
    lib.wkv6_segment_summary_for_scan.restype = ctypes.c_int
    lib.wkv6_segment_summary_for_scan.argtypes = [pp, vp, vp, vp, ctypes.c_int, i32, vp, vp, vp]
    lib.wkv6_sum_rows.restype = ctypes.c_int
    lib.wkv6_sum_rows.argtypes = [vp, ctypes.c_int64, ctypes.c_int64, vp, vp]
    lib.wkv6_state_scan.restype = ctypes.c_int
    lib.wkv6_state_scan.argtypes = [i32, i32, i32, i32, vp, vp, vp, vp, vp, ctypes.c_int, vp]
    lib.wkv6_backward_seeded.restype = ctypes.c_int
    lib.wkv6_backward_seeded.argtypes = [pp] + [vp] * 11 + [vp, vp, vp, sz, vp]
    i64 = ctypes.c_int64
    lib.wkv6_groupnorm_gate_forward.restype = ctypes.c_int
    lib.wkv6_groupnorm_gate_forward.argtypes = [i64, i32, i32, i32, ctypes.c_float, vp, vp, vp, vp, vp, vp]
    lib.wkv6_groupnorm_gate_backward.restype = ctypes.c_int
    lib.wkv6_groupnorm_gate_backward.argtypes = [i64, i32, i32, i32, ctypes.c_float] + [vp] * 10 + [sz, vp]
    lib.wkv6_groupnorm_silu_gate_forward.restype = ctypes.c_int
    lib.wkv6_groupnorm_silu_gate_forward.argtypes = [i64, i32, i32, i32, ctypes.c_float, vp, vp, vp, vp, vp, vp]
    lib.wkv6_groupnorm_silu_gate_backward.restype = ctypes.c_int
    lib.wkv6_groupnorm_silu_gate_backward.argtypes = [i64, i32, i32, i32, ctypes.c_float] + [vp] * 10 + [sz, vp]
    lib.wkv6_groupnorm_gate_workspace_bytes.restype = sz
    lib.wkv6_groupnorm_gate_workspace_bytes.argtypes = [i64, i32, i32]
    lib.wkv6_shift_mix_forward.restype = ctypes.c_int
    lib.wkv6_shift_mix_forward.argtypes = [i32] * 6 + [vp, vp, vp, vp]
    lib.wkv6_shift_mix_backward.restype = ctypes.c_int
    lib.wkv6_shift_mix_backward.argtypes = [i32] * 6 + [vp] * 6 + [sz, vp]
    lib.wkv6_shift_mix_workspace_bytes.restype = sz
    lib.wkv6_shift_mix_workspace_bytes.argtypes = [i32] * 4
    for name, nptr in (("wkv6_relu_sq_forward", 2), ("wkv6_relu_sq_backward", 3), ("wkv6_sigmoid_mul_forward", 3),
                       ("wkv6_sigmoid_mul_backward", 5)):
        fn = getattr(lib, name)
        fn.restype = ctypes.c_int
        fn.argtypes = [i64, i32] + [vp] * nptr + [vp]
    lib.wkv6_copy_2d_async.restype = ctypes.c_int
    lib.wkv6_copy_2d_async.argtypes = [vp, sz, vp, sz, sz, sz, i32, vp]
    lib.wkv6_xla_buffer_bytes.restype = sz
    lib.wkv6_xla_buffer_bytes.argtypes = [ctypes.c_char_p, sz, ctypes.c_int]
    for name in ("wkv6_xla_forward", "wkv6_xla_backward", "wkv6_xla_forward_with_state", "wkv6_xla_forward_ckpt",
                 "wkv6_xla_backward_ws"):
        fn = getattr(lib, name)
        fn.restype = ctypes.c_int
        fn.argtypes = [vp, ctypes.POINTER(vp), ctypes.c_char_p, sz]
    lib.wkv6_xla_descriptor.restype = ctypes.c_int
    lib.wkv6_xla_descriptor.argtypes = [ctypes.c_int] * 7 + [ctypes.c_char_p, sz]
    lib.wkv6_xla_target.restype = vp
    lib.wkv6_xla_target.argtypes = [ctypes.c_int]
    return lib


lib = _load()


def xla_descriptor(B, T, C, H, S, x_type, y_type) -> bytes:
    """The 28-byte opaque blob of the legacy custom calls (replaces gpu_ops.create_rwkv_descriptor)."""
    buf = ctypes.create_string_buffer(32)
    n = lib.wkv6_xla_descriptor(B, T, C, H, int(bool(S)), x_type, y_type, buf, 32)
    if n <= 0:
        raise WKV6Error(n, lib.wkv6_last_error().decode())
    return buf.raw[:n]


def check(rc: int) -> None:
    if rc != 0:
        raise WKV6Error(rc, lib.wkv6_last_error().decode())
