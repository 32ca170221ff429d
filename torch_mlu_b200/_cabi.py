"""ctypes binding of libsdpa_b200.so (the C ABI declared in include/sdpa_b200.h).

The struct below mirrors ``sdpa_b200_params`` field for field. There is no fallback: if the
shared library is missing or a call returns a non-zero status, the caller gets an exception.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint64, c_void_p

LIB_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib")
LIB_PATH = os.path.join(LIB_DIR, "libsdpa_b200.so")

OK, INVALID_ARG, UNSUPPORTED, LAUNCH_FAILED, DEVICE_TIMEOUT, NO_DEVICE = range(6)
KERNEL_AUTO, KERNEL_PREFILL, KERNEL_DECODE = 0, 1, 2
DTYPE_BF16, DTYPE_F16 = 0, 1

# every symbol include/sdpa_b200.h declares
EXPORTED_SYMBOLS = (
    "sdpa_b200_version",
    "sdpa_b200_status_string",
    "sdpa_b200_last_error",
    "sdpa_b200_fwd_workspace_bytes",
    "sdpa_b200_bwd_workspace_bytes",
    "sdpa_b200_fwd",
    "sdpa_b200_bwd",
    "sdpa_b200_read_device_status",
    "sdpa_b200_selftest_wait_timeout",
    "sdpa_b200_decode_static",
    "sdpa_b200_merge_partial",
    "sdpa_b200_dropout_keep_mask",
    "sdpa_b200_dropout_keep_mask_varlen",
    "sdpa_b200_transpose_bias",
    "sdpa_b200_launch_count",
)
STATIC_SCRATCH_BYTES = 16 << 20


class SdpaParams(ctypes.Structure):
    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p),
        ("out", c_void_p), ("lse", c_void_p),
        ("dout", c_void_p), ("dq", c_void_p), ("dk", c_void_p), ("dv", c_void_p),
        ("cu_seqlens_q", c_void_p), ("cu_seqlens_k", c_void_p),
        ("batch", c_int32), ("heads_q", c_int32), ("heads_kv", c_int32), ("head_dim", c_int32),
        ("max_seqlen_q", c_int32), ("max_seqlen_k", c_int32),
        ("total_q", c_int32), ("total_k", c_int32),
        ("q_batch_stride", c_int64), ("q_head_stride", c_int64), ("q_row_stride", c_int64),
        ("k_batch_stride", c_int64), ("k_head_stride", c_int64), ("k_row_stride", c_int64),
        ("v_batch_stride", c_int64), ("v_head_stride", c_int64), ("v_row_stride", c_int64),
        ("o_batch_stride", c_int64), ("o_head_stride", c_int64), ("o_row_stride", c_int64),
        ("do_batch_stride", c_int64), ("do_head_stride", c_int64), ("do_row_stride", c_int64),
        ("dq_batch_stride", c_int64), ("dq_head_stride", c_int64), ("dq_row_stride", c_int64),
        ("dk_batch_stride", c_int64), ("dk_head_stride", c_int64), ("dk_row_stride", c_int64),
        ("dv_batch_stride", c_int64), ("dv_head_stride", c_int64), ("dv_row_stride", c_int64),
        ("softmax_scale", c_float), ("dropout_p", c_float),
        ("is_causal", c_int32), ("dtype", c_int32), ("kernel", c_int32), ("num_splits", c_int32),
        ("keep_rows", c_void_p), ("keep_cols", c_void_p),
        ("bias", c_void_p), ("bias_batch_stride", c_int64), ("bias_head_stride", c_int64), ("bias_row_stride", c_int64),
        ("dbias", c_void_p), ("dbias_batch_stride", c_int64), ("dbias_head_stride", c_int64), ("dbias_row_stride", c_int64),
        ("bias_t", c_void_p), ("bias_t_batch_stride", c_int64), ("bias_t_head_stride", c_int64), ("bias_t_row_stride", c_int64),
        ("deterministic", c_int32), ("sm_margin", c_int32),
        ("device_status", c_void_p),
    ]


class SdpaError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, status: int, text: str):
        super().__init__(text)
        self.status = status


_lib = None


def load() -> ctypes.CDLL:
    """dlopen the in-tree library; raise (never fall back) when it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m torch_mlu_b200.build` "
            "(there is no CPU or eager fallback for this path)"
        )
    lib = ctypes.CDLL(LIB_PATH)
    lib.sdpa_b200_version.restype = c_int
    lib.sdpa_b200_status_string.restype = c_char_p
    lib.sdpa_b200_status_string.argtypes = [c_int]
    lib.sdpa_b200_last_error.restype = c_char_p
    lib.sdpa_b200_launch_count.restype = c_uint64
    for name in ("sdpa_b200_fwd_workspace_bytes", "sdpa_b200_bwd_workspace_bytes"):
        fn = getattr(lib, name)
        fn.restype = c_int
        fn.argtypes = [POINTER(SdpaParams), POINTER(c_size_t)]
    for name in ("sdpa_b200_fwd", "sdpa_b200_bwd"):
        fn = getattr(lib, name)
        fn.restype = c_int
        fn.argtypes = [POINTER(SdpaParams), c_void_p, c_size_t, c_void_p]
    lib.sdpa_b200_read_device_status.restype = c_int
    lib.sdpa_b200_read_device_status.argtypes = [c_void_p, c_void_p, POINTER(c_int)]
    lib.sdpa_b200_selftest_wait_timeout.restype = c_int
    lib.sdpa_b200_selftest_wait_timeout.argtypes = [c_void_p, ctypes.c_uint32, c_void_p]
    lib.sdpa_b200_decode_static.restype = c_int
    lib.sdpa_b200_decode_static.argtypes = [POINTER(SdpaParams), c_void_p]
    lib.sdpa_b200_merge_partial.restype = c_int
    lib.sdpa_b200_merge_partial.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32,
                                            c_int32, c_int64, c_int64, c_int64, c_void_p]
    lib.sdpa_b200_dropout_keep_mask.restype = c_int
    lib.sdpa_b200_dropout_keep_mask.argtypes = [c_uint64, c_uint64, c_float, c_int32, c_int32, c_int32, c_int32, c_int32,
                                                c_void_p, c_void_p, c_void_p]
    lib.sdpa_b200_dropout_keep_mask_varlen.restype = c_int
    lib.sdpa_b200_dropout_keep_mask_varlen.argtypes = [c_uint64, c_uint64, c_float, c_int32, c_int32, c_void_p, c_void_p, c_int32,
                                                       c_int32, c_int32, c_int32, c_int32, c_void_p, c_void_p, c_void_p]
    lib.sdpa_b200_transpose_bias.restype = c_int
    lib.sdpa_b200_transpose_bias.argtypes = [c_void_p, c_int64, c_int64, c_int64, c_int32, c_int32, c_int32, c_int32, c_void_p,
                                             c_int64, c_void_p]
    _lib = lib
    return lib


def check(status: int, what: str) -> None:
    if status != OK:
        lib = load()
        kind = lib.sdpa_b200_status_string(status).decode()
        detail = lib.sdpa_b200_last_error().decode()
        raise SdpaError(status, f"{what}: {kind}: {detail}")


def launch_count() -> int:
    return int(load().sdpa_b200_launch_count())
