"""CPU-side checks of the C-ABI boundary: the library loads, exports every symbol the header
declares, the ctypes mirror of the params struct matches the C layout, and argument validation
answers with status codes (no compute is launched here)."""
import ctypes
import os
import re
import subprocess

import pytest
import torch

from torch_mlu_b200 import _cabi, ops

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "sdpa_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    return re.findall(r"SDPA_B200_API\s+[\w\s\*]+?\b(sdpa_b200_\w+)\s*\(", text)


def test_header_symbols_are_exported(native_lib):
    names = declared_symbols()
    assert set(names) == set(_cabi.EXPORTED_SYMBOLS), names
    for n in names:
        assert hasattr(native_lib, n), f"{n} declared in the header but not exported"
    assert native_lib.sdpa_b200_version() == 108
    assert native_lib.sdpa_b200_status_string(1) == b"invalid argument"


def test_ctypes_struct_matches_c_layout(tmp_path):
    fields = [f[0] for f in _cabi.SdpaParams._fields_]
    prog = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{HEADER}"', "int main(void){",
            'printf("%zu\\n", sizeof(sdpa_b200_params));']
    prog += [f'printf("%zu\\n", offsetof(sdpa_b200_params, {f}));' for f in fields]
    prog += ["return 0;}"]
    src = tmp_path / "layout.c"
    src.write_text("\n".join(prog))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", str(src), "-o", str(exe)], check=True)
    vals = [int(x) for x in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()]
    assert vals[0] == ctypes.sizeof(_cabi.SdpaParams)
    for f, off in zip(fields, vals[1:]):
        assert getattr(_cabi.SdpaParams, f).offset == off, f


def _valid_params():
    p = _cabi.SdpaParams()
    p.q = p.k = p.v = p.out = p.lse = 4096  # never dereferenced on the host
    p.batch, p.heads_q, p.heads_kv, p.head_dim = 2, 8, 2, 128
    p.max_seqlen_q = p.max_seqlen_k = 256
    for t in "qkvo":
        setattr(p, f"{t}_batch_stride", 8 * 256 * 128)
        setattr(p, f"{t}_head_stride", 256 * 128)
        setattr(p, f"{t}_row_stride", 128)
    p.softmax_scale = 0.088
    return p


def _ws_bytes(lib, p, bwd=False):
    n = ctypes.c_size_t(0)
    fn = lib.sdpa_b200_bwd_workspace_bytes if bwd else lib.sdpa_b200_fwd_workspace_bytes
    return fn(ctypes.byref(p), ctypes.byref(n)), n.value


def test_workspace_query_and_validation_codes(native_lib):
    lib = native_lib
    st, n = _ws_bytes(lib, _valid_params())
    assert st == _cabi.OK and n >= 256

    def expect(mutate, status, needle):
        p = _valid_params()
        mutate(p)
        st, _ = _ws_bytes(lib, p)
        assert st == status, (st, lib.sdpa_b200_last_error())
        assert needle in lib.sdpa_b200_last_error().decode(), lib.sdpa_b200_last_error()

    expect(lambda p: setattr(p, "heads_kv", 3), _cabi.INVALID_ARG, "must divide number of heads in query")
    expect(lambda p: setattr(p, "head_dim", 100), _cabi.INVALID_ARG, "multiple of 8")
    expect(lambda p: setattr(p, "head_dim", 264), _cabi.INVALID_ARG, "at most 256")
    def wide_with_bias(p):
        p.head_dim, p.bias = 192, 4096
    expect(wide_with_bias, _cabi.UNSUPPORTED, "without a bias")
    expect(lambda p: setattr(p, "dropout_p", 0.1), _cabi.INVALID_ARG, "needs keep_rows")
    expect(lambda p: setattr(p, "dropout_p", 1.0), _cabi.INVALID_ARG, "inside (0, 1)")
    expect(lambda p: setattr(p, "keep_rows", 4096), _cabi.INVALID_ARG, "must be NULL when dropout_p is 0")
    expect(lambda p: setattr(p, "dtype", 3), _cabi.UNSUPPORTED, "bf16")
    expect(lambda p: setattr(p, "max_seqlen_k", 0), _cabi.INVALID_ARG, "sequence lengths must be positive")
    expect(lambda p: setattr(p, "softmax_scale", 0.0), _cabi.INVALID_ARG, "softmax_scale")
    expect(lambda p: setattr(p, "q", 0), _cabi.INVALID_ARG, "q is NULL")
    expect(lambda p: setattr(p, "k", 4100), _cabi.INVALID_ARG, "16-byte aligned")
    expect(lambda p: setattr(p, "q_row_stride", 130), _cabi.INVALID_ARG, "strides")
    expect(lambda p: setattr(p, "cu_seqlens_q", 4096), _cabi.INVALID_ARG, "both be given")
    expect(lambda p: setattr(p, "lse", 0), _cabi.INVALID_ARG, "lse is NULL")

    st = lib.sdpa_b200_fwd_workspace_bytes(None, ctypes.byref(ctypes.c_size_t()))
    assert st == _cabi.INVALID_ARG


def test_decode_workspace_grows_with_splits(native_lib):
    p = _valid_params()
    p.max_seqlen_q, p.max_seqlen_k, p.kernel = 1, 32768, _cabi.KERNEL_DECODE
    p.num_splits = 1
    _, n1 = _ws_bytes(native_lib, p)
    p.num_splits = 16
    _, n16 = _ws_bytes(native_lib, p)
    assert n1 == 256 and n16 >= 256 + 2 * 8 * 16 * 129 * 4


def test_decode_static_refuses_what_it_has_no_kernel_for_before_touching_a_device(native_lib):
    """sdpa_b200_decode_static launches the 64- and 128-column split-KV kernels only: any other head dim, dropout,
    a bias, packed tensors, more than one query row and partials beyond the built-in array are turned away by
    status code. All of these answers come before the device check, so they are the same with and without a GPU."""
    lib = native_lib

    def decode_params():
        p = _valid_params()
        p.max_seqlen_q, p.max_seqlen_k, p.kernel = 1, 4096, _cabi.KERNEL_DECODE
        return p

    def expect(mutate, status, needle):
        p = decode_params()
        mutate(p)
        st = lib.sdpa_b200_decode_static(ctypes.byref(p), None)
        assert st == status, (st, lib.sdpa_b200_last_error())
        assert needle in lib.sdpa_b200_last_error().decode(), lib.sdpa_b200_last_error()

    expect(lambda p: setattr(p, "head_dim", 96), _cabi.UNSUPPORTED, "head_dim 64 and 128 only")
    expect(lambda p: setattr(p, "head_dim", 32), _cabi.UNSUPPORTED, "head_dim 64 and 128 only")
    expect(lambda p: setattr(p, "bias", 4096), _cabi.UNSUPPORTED, "bias")

    def dropout_auto(p):
        p.kernel, p.dropout_p, p.keep_rows = _cabi.KERNEL_AUTO, 0.1, 4096
    expect(dropout_auto, _cabi.UNSUPPORTED, "no dropout")
    expect(lambda p: setattr(p, "dropout_p", 0.1), _cabi.UNSUPPORTED, "no dropout")

    def bias_auto(p):
        p.kernel, p.bias = _cabi.KERNEL_AUTO, 4096
    expect(bias_auto, _cabi.UNSUPPORTED, "bias")
    expect(lambda p: setattr(p, "kernel", _cabi.KERNEL_PREFILL), _cabi.UNSUPPORTED, "decode kernel only")
    expect(lambda p: setattr(p, "max_seqlen_q", 4), _cabi.UNSUPPORTED, "seqlen_q == 1")

    def packed(p):
        p.cu_seqlens_q = p.cu_seqlens_k = 4096
        p.total_q, p.total_k = 2, 8192
    expect(packed, _cabi.UNSUPPORTED, "dense tensors only")

    def too_large(p):
        p.batch, p.heads_q, p.num_splits = 64, 32, 64
    expect(too_large, _cabi.INVALID_ARG, "more than the")
    # the ordinary forward entry point gives the same answer for the head dim
    p = decode_params()
    p.head_dim = 96
    assert lib.sdpa_b200_fwd(ctypes.byref(p), 4096, 1 << 24, None) == _cabi.UNSUPPORTED


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU answer")
def test_compute_calls_refuse_without_a_gpu(native_lib):
    """No CPU fallback: with valid arguments but no device the call reports NO_DEVICE."""
    p = _valid_params()
    st = native_lib.sdpa_b200_fwd(ctypes.byref(p), 4096, 1 << 20, None)
    assert st == _cabi.NO_DEVICE
    assert b"no CPU path" in native_lib.sdpa_b200_last_error() or b"sm_100" in native_lib.sdpa_b200_last_error()
    # and a too-small / misaligned workspace is refused before the device is touched
    assert native_lib.sdpa_b200_fwd(ctypes.byref(p), 4096, 16, None) == _cabi.INVALID_ARG
    assert native_lib.sdpa_b200_fwd(ctypes.byref(p), 4100, 1 << 20, None) == _cabi.INVALID_ARG


def test_host_mirror_rejects_what_the_reference_rejects():
    """Error behaviour of the operator mirror on host tensors (attention.cpp:70-100,
    FlashAttention_internal.cpp:74-127)."""
    q = torch.zeros(1, 2, 16, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA device"):
        ops._scaled_dot_product_flash_attention(q, q, q)
    with pytest.raises(RuntimeError, match="4-dimensional"):
        ops._scaled_dot_product_flash_attention(q[0], q[0], q[0])
    with pytest.raises(RuntimeError, match="same number of heads"):
        ops._scaled_dot_product_flash_attention(q, q[:, :1], q[:, :1])
    with pytest.raises(RuntimeError, match="same sequence length"):
        ops._scaled_dot_product_flash_attention(q, q, q[:, :, :8])
    with pytest.raises(RuntimeError, match="dropout_p must be inside"):
        ops._scaled_dot_product_flash_attention(q, q, q, dropout_p=1.0)
    cu = torch.tensor([0, 16], dtype=torch.int64)
    p = q[0].transpose(0, 1)
    with pytest.raises(RuntimeError, match="int32"):
        ops._flash_attention_forward(p, p, p, cu, cu, 16, 16, 0.0, False, False)
    assert ops.calculate_scale(q, None) == pytest.approx(128 ** -0.5)
    assert ops.calculate_scale(q, 0.5) == 0.5


def test_helper_entry_points_check_their_arguments_before_touching_a_device(native_lib):
    """sdpa_b200_dropout_keep_mask[_varlen] and sdpa_b200_transpose_bias refuse bad arguments with INVALID_ARG
    and a message; none of these checks needs a GPU."""
    lib = native_lib
    err = lambda: lib.sdpa_b200_last_error().decode()
    assert lib.sdpa_b200_dropout_keep_mask(1, 0, 0.1, 1, 1, 128, 128, 0, None, None, None) == _cabi.INVALID_ARG
    assert "16-byte aligned" in err()
    assert lib.sdpa_b200_dropout_keep_mask(1, 0, 0.1, 1, 1, 128, 128, 0, 4096, 8192 + 8, None) == _cabi.INVALID_ARG
    assert lib.sdpa_b200_dropout_keep_mask(1, 0, 1.5, 1, 1, 128, 128, 0, 4096, 8192, None) == _cabi.INVALID_ARG
    assert "inside (0, 1)" in err()
    assert lib.sdpa_b200_dropout_keep_mask(1, 0, 0.1, 70000, 1, 128, 128, 0, 4096, 8192, None) == _cabi.INVALID_ARG
    assert "65535" in err()
    assert lib.sdpa_b200_dropout_keep_mask_varlen(1, 0, 0.1, 2, 1, None, None, 10, 10, 8, 8, 0, 4096, 8192, None) == _cabi.INVALID_ARG
    assert lib.sdpa_b200_transpose_bias(4096, 0, 0, 0, 1, 1, 64, 64, 8192, 64, None) == _cabi.INVALID_ARG
    assert "non-zero row stride" in err()
    assert lib.sdpa_b200_transpose_bias(4096, 0, 0, 64, 1, 1, 64, 64, 8192, 60, None) == _cabi.INVALID_ARG
    assert "out_row_stride" in err()
