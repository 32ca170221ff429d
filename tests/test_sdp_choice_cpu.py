"""Backend choice and its error texts, after the reference's TestSDPAThrowException
(test/torch_ops/test_scaled_dot_product_attention.py:243-479): with only the flash backend enabled,
an input the fused kernel cannot take produces the matching UserWarning and a RuntimeError."""
import warnings

import pytest
import torch

from torch_mlu_b200 import backends, sdp_choice
from torch_mlu_b200.backends import SDPBackend

FLASH_ONLY = dict(enable_flash=True, enable_math=False, enable_mem_efficient=False)


def make(size, dtype=torch.bfloat16):
    return torch.randn(size).to(dtype)


def expect_rejected(pattern, q, k, v, mask=None, dropout_p=0.0):
    with backends.sdp_kernel(**FLASH_ONLY):
        with pytest.warns(UserWarning, match=pattern):
            with pytest.raises(RuntimeError, match="No available kernel"):
                sdp_choice.scaled_dot_product_attention(q, k, v, mask, dropout_p, False)


def test_no_backend_enabled_is_an_error():
    q = make((2, 2, 8, 64))
    with backends.sdp_kernel(enable_flash=False, enable_math=False, enable_mem_efficient=False):
        assert sdp_choice._fused_sdp_choice(q, q, q) == int(SDPBackend.ERROR)
        with pytest.raises(RuntimeError, match="No viable backend"):
            sdp_choice.scaled_dot_product_attention(q, q, q)


def test_non_4d_inputs():
    q = make((2, 8, 64))
    expect_rejected("Both fused kernels requires query, key and value to be 4 dimensional", q, q, q)


def test_mismatched_batch_or_heads():
    q, k = make((2, 4, 8, 64)), make((2, 2, 8, 64))
    expect_rejected("both fused kernels require query, key and value to have the same batch_size and num_heads", q, k, k)


def test_attn_mask_present():
    q = make((2, 2, 3, 64))
    expect_rejected("Flash Attention does not support non-null attn_mask.", q, q, q, torch.ones(2, 2, 3, 3, dtype=q.dtype))


def test_bad_head_dim():
    q = make((2, 2, 3, 40))
    expect_rejected("Flash attention requires q,k,v to have the same last dimension", q, q, q)
    q = make((2, 2, 3, 264))
    expect_rejected("256>=query.size", q, q, q)


def test_zero_sequence_length():
    q, k = make((2, 2, 0, 64)), make((2, 2, 3, 64))
    expect_rejected("Both fused kernels do not support zero seq_len_q or seq_len_kv.", q, k, k)


def test_last_dim_stride():
    q = make((2, 2, 64, 3)).transpose(-1, -2)  # [2,2,3,64] with stride(-1) == 3
    k = make((2, 2, 3, 64))
    expect_rejected("Both fused kernels require the last dimension of the input to have stride 1", q, k, k)


def test_cpu_tensors_and_dtype():
    q = make((2, 2, 3, 64))
    expect_rejected("only runs on an sm_100 CUDA device", q, q, q)


def test_math_backend_is_the_fallback_when_enabled():
    q = make((1, 2, 8, 64), torch.float32)
    with backends.sdp_kernel(enable_flash=True, enable_math=True, enable_mem_efficient=False):
        with warnings.catch_warnings():
            warnings.simplefilter("error")
            assert sdp_choice._fused_sdp_choice(q, q, q) == int(SDPBackend.MATH)
            out = sdp_choice.scaled_dot_product_attention(q, q, q, is_causal=True)
    ref = torch.nn.functional.scaled_dot_product_attention(q, q, q, is_causal=True)
    assert torch.allclose(out, ref, atol=1e-6)


def test_memory_efficient_backend_takes_a_mask_that_broadcasts():
    q = make((2, 2, 3, 64))
    with backends.sdp_kernel(enable_flash=False, enable_math=False, enable_mem_efficient=True):
        with pytest.warns(UserWarning, match="does not broadcast to the attention scores"):
            with pytest.raises(RuntimeError, match="No available kernel"):
                sdp_choice.scaled_dot_product_attention(q, q, q, torch.ones(2, 2, 5, 3, dtype=q.dtype))
        with pytest.warns(UserWarning, match="Flash attention has been runtime disabled"):
            with pytest.raises(RuntimeError, match="No available kernel"):
                sdp_choice.scaled_dot_product_attention(q, q, q)  # CPU tensors: the device check fails too


def test_priority_order_follows_the_reference_heuristics():
    """sdp_utils.cpp:8-50, on tensor metadata only."""
    F, E, M = SDPBackend.FLASH_ATTENTION, SDPBackend.EFFICIENT_ATTENTION, SDPBackend.MATH
    z = lambda *s: torch.zeros(*s, dtype=torch.bfloat16)
    order = sdp_choice.priority_order
    assert order(z(1, 2, 64, 64), z(1, 2, 64, 64), z(1, 2, 64, 64)) == (F, E, M)        # few threads, short queries
    assert order(z(1, 2, 256, 64), z(1, 2, 256, 64), z(1, 2, 256, 64)) == (E, F, M)     # few threads, long queries
    assert order(z(8, 16, 256, 64), z(8, 16, 256, 64), z(8, 16, 256, 64)) == (F, E, M)  # 128 (batch, head) units
    assert order(z(8, 16, 256, 128), z(8, 16, 256, 128), z(8, 16, 256, 128)) == (E, F, M)  # head_dim 128, inference
    q = z(8, 16, 2048, 128).requires_grad_(True)
    assert order(q, q, q) == (F, E, M)              # training: 6 * 128 <= 2048
    q = z(8, 16, 512, 128).requires_grad_(True)
    assert order(q, q, q) == (E, F, M)              # training: 6 * 128 > 512
    with torch.no_grad():
        assert order(q, q, q) == (E, F, M)          # grad mode off: the inference rule (head_dim 128)
    assert order(z(2, 64, 64), z(2, 64, 64), z(2, 64, 64)) == (F, E, M)  # not 4-dimensional
