"""Backend choice for scaled_dot_product_attention, mirroring the reference's
``cnnl__fused_sdp_choice`` / ``select_sdp_backend``
(torch_mlu/csrc/aten/operators/cnnl/transformers/_fused_sdp_choice.cpp:38-56, sdp_utils.cpp:97-147).

Same decision procedure and the same warning / error texts for the constraints that carry over
(sdp_utils.h:99-455): backends in priority order, each with a constraint list; if none qualifies
and math is disabled, every constraint is re-run in debug mode (warnings) and
``RuntimeError("No available kernel.  Aborting execution.")`` is raised. What differs on purpose:
both fused backends run the same kernels here (flash refuses an attn_mask as in the reference; the
memory-efficient one takes it as an additive bias), and the MLU-occupancy heuristics of sdp_utils.h:479-524 (500-series check, split condition, valid-data
ratio) are replaced by what this build needs: an sm_100 CUDA device, and no attn_mask when head_dim exceeds 128.
"""
from __future__ import annotations

import warnings
from typing import Optional

import torch

from . import backends
from .backends import SDPBackend


def _warn(debug: bool, msg: str) -> None:
    if debug:
        warnings.warn(msg, UserWarning, stacklevel=4)


def _check_runtime_disabled_flash(q, k, v, mask, debug):  # sdp_utils.h:99-109
    if not backends.flash_sdp_enabled():
        _warn(debug, "Flash attention has been runtime disabled.")
        return False
    return True


def _check_tensor_shapes(q, k, v, mask, debug):  # sdp_utils.h:125-143
    if not (q.dim() == k.dim() == v.dim() == 4):
        _warn(debug, "Both fused kernels requires query, key and value to be 4 dimensional, but got Query dim: "
                     f"{q.dim()}, Key dim: {k.dim()}, Value dim: {v.dim()} instead.")
        return False
    return True


def _check_batch_size_and_num_heads(q, k, v, mask, debug, allow_gqa=False):  # sdp_utils.h:159-219
    same_batch = q.size(0) == k.size(0) == v.size(0)
    if allow_gqa:
        same_heads = k.size(1) == v.size(1) and k.size(1) > 0 and q.size(1) % k.size(1) == 0
    else:
        same_heads = q.size(1) == k.size(1) == v.size(1)
    if not (same_batch and same_heads):
        _warn(debug, "For dense inputs, both fused kernels require query, key and value to have the same batch_size "
                     f"and num_heads. Query.sizes(): {list(q.shape)}, Key sizes(): {list(k.shape)}, "
                     f"Value sizes(): {list(v.shape)} instead. To broadcast dense inputs, try using unsqueeze and "
                     "expand_to before passing them into the kernel.")
        return False
    return True


def _check_for_attn_mask(q, k, v, mask, debug):  # sdp_utils.h:221-229
    if mask is not None:
        _warn(debug, "Flash Attention does not support non-null attn_mask.")
        return False
    return True


def _check_head_dim_size(q, k, v, mask, debug):  # sdp_utils.h:231-255
    d = q.size(-1)
    same = d == k.size(-1) == v.size(-1)
    if not (same and 256 >= d >= 64 and d % 8 == 0):
        _warn(debug, "Flash attention requires q,k,v to have the same last dimension.256>=query.size(-1)>=64."
                     "Flash attention requires last dimension of inputs to be divisible by 8."
                     f" Got Query.size(-1): {d}, Key.size(-1): {k.size(-1)}, Value.size(-1): {v.size(-1)} instead.")
        return False
    return True


def _check_nonzero_sequence_lengths(q, k, v, mask, debug):  # sdp_utils.h:371-392
    if q.size(-2) == 0 or k.size(-2) == 0:
        _warn(debug, "Both fused kernels do not support zero seq_len_q or seq_len_kv.")
        return False
    return True


def _check_last_dim_stride_equals_1(q, k, v, mask, debug):  # sdp_utils.h:394-431
    ok = q.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1 and (mask is None or mask.stride(-1) == 1)
    if not ok:
        tail = f", Attn_mask.stride(-1): {mask.stride(-1)}" if mask is not None else ""
        _warn(debug, "Both fused kernels require the last dimension of the input to have stride 1. "
                     f"Got Query.stride(-1): {q.stride(-1)}, Key.stride(-1): {k.stride(-1)}, "
                     f"Value.stride(-1): {v.stride(-1)}{tail} instead.")
        return False
    return True


def _check_fused_kernel_device_support(q, k, v, mask, debug):  # stands where sdp_utils.h:479-524 stood
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        _warn(debug, "The fused kernel only runs on an sm_100 CUDA device. Attempting to run on "
                     f"{q.device.type}.")
        return False
    if torch.cuda.get_device_capability(q.device)[0] != 10:
        _warn(debug, "The fused kernel only supports sm_100 (B200). Attempting to run on "
                     f"{torch.cuda.get_device_name(q.device)}.")
        return False
    if q.size(-1) > 128 and mask is not None:
        _warn(debug, "This build runs head dims above 128 without an attn_mask (the additive bias is built for head_dim up "
                     f"to 128). Got Query.size(-1): {q.size(-1)}.")
        return False
    return True


def _check_tensor_dtype(q, k, v, mask, debug):  # sdp_utils.h:433-455
    if not (q.dtype == k.dtype == v.dtype and q.dtype in (torch.float16, torch.bfloat16)):
        _warn(debug, "Expected query, key and value to all be of dtype: {Half, BFloat16}. Got "
                     f"Query dtype: {q.dtype}, Key dtype: {k.dtype}, and Value dtype: {v.dtype} instead.")
        return False
    return True


_FLASH_CONSTRAINTS = (
    _check_runtime_disabled_flash,
    _check_tensor_shapes,
    _check_batch_size_and_num_heads,
    _check_for_attn_mask,
    _check_head_dim_size,
    _check_nonzero_sequence_lengths,
    _check_last_dim_stride_equals_1,
    _check_fused_kernel_device_support,
    _check_tensor_dtype,
)


def use_flash_attention(query, key, value, attn_mask=None, debug: bool = False) -> bool:
    """sdp_utils.cpp:52-72."""
    return all(c(query, key, value, attn_mask, debug) for c in _FLASH_CONSTRAINTS)


def _check_runtime_disabled_mem_efficient(q, k, v, mask, debug):  # sdp_utils.h:111-123
    if not backends.mem_efficient_sdp_enabled():
        _warn(debug, "Memory efficient attention has been runtime disabled.")
        return False
    return True


def _check_mask_for_mem_efficient(q, k, v, mask, debug):
    # the bias joins the scores inside the kernel: it has to broadcast to [B, H, Lq, Lk]
    if mask is not None:
        try:
            torch.broadcast_shapes(tuple(mask.shape), (q.size(0), q.size(1), q.size(2), k.size(2)))
        except RuntimeError:
            _warn(debug, f"attn_mask of shape {tuple(mask.shape)} does not broadcast to the attention scores.")
            return False
        if mask.dim() > 4:
            _warn(debug, "attn_mask must have at most 4 dimensions.")
            return False
    return True


_MEM_EFFICIENT_CONSTRAINTS = (
    _check_runtime_disabled_mem_efficient,
    _check_tensor_shapes,
    _check_batch_size_and_num_heads,
    _check_mask_for_mem_efficient,
    _check_head_dim_size,
    _check_nonzero_sequence_lengths,
    _check_last_dim_stride_equals_1,
    _check_fused_kernel_device_support,
    _check_tensor_dtype,
)


def use_mem_efficient_attention(query, key, value, attn_mask=None, debug: bool = False) -> bool:
    """sdp_utils.cpp:74-95."""
    return all(c(query, key, value, attn_mask, debug) for c in _MEM_EFFICIENT_CONSTRAINTS)


def priority_order(query, key, value):
    """The order in which the backends are tried (sdp_utils.cpp:8-50): flash, memory efficient, math - except that the
    memory-efficient operator goes first for nested inputs, for inference with head_dim 128 or with few (batch x head)
    units and long queries, and for training when 6 * batch * heads exceeds the query length. Here both fused
    operators run the same kernels, so the order only decides which operator (and which causal alignment for
    Lq != Lk) a call lands on - as it does in the reference."""
    default_order = (SDPBackend.FLASH_ATTENTION, SDPBackend.EFFICIENT_ATTENTION, SDPBackend.MATH)
    efficient_first = (SDPBackend.EFFICIENT_ATTENTION, SDPBackend.FLASH_ATTENTION, SDPBackend.MATH)
    if query.is_nested or key.is_nested or value.is_nested:
        return efficient_first
    if query.dim() != 4:
        return default_order
    batch_size, num_heads, query_lengths, head_dim = query.shape
    if batch_size > 0:
        threads_flash = batch_size * num_heads
        threads_cutlass = threads_flash * (query_lengths // 64)
        more_threads_cutlass = (threads_cutlass // 2) >= threads_flash
        small_threads_flash = threads_flash < 60
        large_head_dim = max(head_dim, key.size(3) if key.dim() == 4 else head_dim) == 128
        requires_grad = torch.is_grad_enabled() and (query.requires_grad or key.requires_grad or value.requires_grad)
        if requires_grad:
            if 6 * threads_flash > query_lengths:
                return efficient_first
        elif (small_threads_flash and more_threads_cutlass) or large_head_dim:
            return efficient_first
    return default_order


def _fused_sdp_choice(query, key, value, attn_mask=None, dropout_p: float = 0.0, is_causal: bool = False,
                      *, scale: Optional[float] = None) -> int:
    """Returns the SDPBackend value (int) the call would use, or raises like the reference (select_sdp_backend,
    sdp_utils.cpp:97-147)."""
    if not (backends.math_sdp_enabled() or backends.flash_sdp_enabled() or backends.mem_efficient_sdp_enabled()):
        return int(SDPBackend.ERROR)
    for backend in priority_order(query, key, value):
        if backend == SDPBackend.FLASH_ATTENTION and use_flash_attention(query, key, value, attn_mask, False):
            return int(SDPBackend.FLASH_ATTENTION)
        if backend == SDPBackend.EFFICIENT_ATTENTION and use_mem_efficient_attention(query, key, value, attn_mask, False):
            return int(SDPBackend.EFFICIENT_ATTENTION)
        if backend == SDPBackend.MATH and backends.math_sdp_enabled():
            return int(SDPBackend.MATH)
    # nothing qualifies: say why, then fail (sdp_utils.cpp:134-146)
    warnings.warn("Memory efficient kernel not used because:", UserWarning, stacklevel=2)
    use_mem_efficient_attention(query, key, value, attn_mask, True)
    warnings.warn("Flash attention kernel not used because:", UserWarning, stacklevel=2)
    use_flash_attention(query, key, value, attn_mask, True)
    raise RuntimeError("No available kernel.  Aborting execution.")


class _EfficientAttention(torch.autograd.Function):
    """Autograd for the memory-efficient operator pair of ops.py (what upstream derivatives.yaml wires for
    _scaled_dot_product_efficient_attention): gradients for query, key, value and a floating-point bias."""

    @staticmethod
    def forward(ctx, query, key, value, bias, dropout_p, is_causal, scale):
        from . import ops
        out, lse, seed, offset = ops._scaled_dot_product_efficient_attention(query, key, value, bias, True, dropout_p, is_causal,
                                                                             scale=scale)
        ctx.save_for_backward(query, key, value, out, lse, seed, offset, *(() if bias is None else (bias,)))
        ctx.args = (dropout_p, is_causal, scale, bias is not None)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        from . import ops
        query, key, value, out, lse, seed, offset, *rest = ctx.saved_tensors
        dropout_p, is_causal, scale, has_bias = ctx.args
        bias = rest[0] if has_bias else None
        need_bias = has_bias and ctx.needs_input_grad[3]
        dq, dk, dv, db = ops._scaled_dot_product_efficient_attention_backward(
            grad_out, query, key, value, bias, out, lse, seed, offset, dropout_p, [True, True, True, need_bias], is_causal,
            scale=scale)
        return dq, dk, dv, (db if need_bias else None), None, None, None


def _mask_to_bias(attn_mask, query):
    """A boolean attn_mask (True = take part) becomes 0 / -inf; a floating-point one is the bias itself."""
    if attn_mask is None:
        return None
    if attn_mask.dtype == torch.bool:
        return torch.zeros_like(attn_mask, dtype=query.dtype).masked_fill(~attn_mask, float("-inf"))
    return attn_mask.to(query.dtype)


def scaled_dot_product_attention(query, key, value, attn_mask=None, dropout_p: float = 0.0, is_causal: bool = False,
                                 scale: Optional[float] = None):
    """F.scaled_dot_product_attention with this package's choice function in front: the flash
    backend runs this library's kernels (through the dispatcher glue, so autograd works), the memory
    efficient one runs them with an attn_mask as additive bias, the math backend is torch's composite
    implementation."""
    choice = _fused_sdp_choice(query, key, value, attn_mask, dropout_p, is_causal, scale=scale)
    if choice == int(SDPBackend.ERROR):
        raise RuntimeError("No viable backend for scaled_dot_product_attention was found.")
    if choice == int(SDPBackend.EFFICIENT_ATTENTION) and attn_mask is not None:
        return _EfficientAttention.apply(query, key, value, _mask_to_bias(attn_mask, query), dropout_p, is_causal, scale)
    if choice == int(SDPBackend.FLASH_ATTENTION) or (
            choice == int(SDPBackend.EFFICIENT_ATTENTION) and (not is_causal or query.size(-2) == key.size(-2))):
        # same kernels, same mask when Lq == Lk: the registered operator also carries autograd
        from . import torch_glue
        torch_glue.load()
        return torch.ops.b200_sdpa._scaled_dot_product_flash_attention(query, key, value, dropout_p, is_causal, False,
                                                                       scale=scale)[0]
    if choice == int(SDPBackend.EFFICIENT_ATTENTION):
        # top-left causal mask with Lq != Lk: the operator mirror, with its own autograd
        return _EfficientAttention.apply(query, key, value, None, dropout_p, is_causal, scale)
    return torch.ops.aten._scaled_dot_product_attention_math(query, key, value, attn_mask, dropout_p, is_causal,
                                                             scale=scale)[0]
