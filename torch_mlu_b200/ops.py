"""Host-side mirror of torch_mlu's attention operator interface, over the C ABI.

Each function keeps the name, argument order, return tuple and error behaviour of the
reference operator it stands for (torch-2.1 schemas, codegen/mlu_functions.yaml:1312-1316):

* ``_scaled_dot_product_flash_attention``           <- cnnl__scaled_dot_product_flash_attention
  (torch_mlu/csrc/aten/operators/cnnl/transformers/attention.cpp:58-159)
* ``_flash_attention_forward``                      <- cnnl__flash_attention_forward (attention.cpp:161-203)
* ``_scaled_dot_product_flash_attention_backward``  <- attention.cpp:205-297
* ``_flash_attention_backward``                     <- cnnl__flash_attention_backward (attention.cpp:299-348)
* ``_scaled_dot_product_efficient_attention[_backward]`` <- attention.cpp:350-391, 510-600, for calls without an
  additive bias (top-left causal convention)

Unlike the reference wrappers, nothing is re-packed: tensors go to the kernels with their
strides (any [B,H,L,D] / [B,L,H,D] view with unit head_dim stride), so the five
``cnnl_contiguous`` copies of attention.cpp:124-129, 260-269 do not exist here.

torch is used for device memory and the current stream only. There is no CPU path: a call
on a machine without the built library or without an sm_100 GPU raises.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional, Tuple

import torch

from . import _cabi, dropout

__all__ = [
    "_scaled_dot_product_flash_attention",
    "_scaled_dot_product_flash_attention_backward",
    "_flash_attention_forward",
    "_flash_attention_backward",
    "decode_attention",
    "calculate_scale",
    "workspace_for",
]

_DECODE_MAX_Q = 1


def calculate_scale(query: torch.Tensor, scale: Optional[float]) -> float:
    """Default softmax scale 1/sqrt(head_dim) (sdp_utils.h:40-47)."""
    return float(scale) if scale is not None else 1.0 / math.sqrt(query.size(-1))


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _check_inputs(*tensors: torch.Tensor) -> None:
    for t in tensors:
        _check(t.is_cuda, "Input tensor must be on a CUDA device (this path has no CPU fallback)")
        # FlashAttention_internal.cpp:74-80
        _check(t.dtype in (torch.bfloat16, torch.float16),
               f"FlashAttention only support fp16 and bf16 data type (got {t.dtype})")
        _check(t.dtype == tensors[0].dtype, "query, key, and value must have the same dtype")
        # FlashAttention_internal.cpp:100-108
        _check(t.stride(-1) == 1, "Input tensor must have contiguous last dimension")


def _stream_ptr(device: Optional[torch.device] = None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _set_strides_bhld(p: _cabi.SdpaParams, prefix: str, t: torch.Tensor) -> None:
    """t is [B, H, L, D] (any strides, unit last)."""
    setattr(p, f"{prefix}_batch_stride", t.stride(0))
    setattr(p, f"{prefix}_head_stride", t.stride(1))
    setattr(p, f"{prefix}_row_stride", t.stride(2))


def _set_strides_thd(p: _cabi.SdpaParams, prefix: str, t: torch.Tensor) -> None:
    """t is packed [total, H, D]."""
    setattr(p, f"{prefix}_batch_stride", 0)
    setattr(p, f"{prefix}_head_stride", t.stride(1))
    setattr(p, f"{prefix}_row_stride", t.stride(0))


class _Workspace:
    """Per-device cache of one growing workspace buffer per stream, and of the device's status word (torch owns
    the memory)."""

    _bufs: dict = {}
    _status: dict = {}

    @classmethod
    def get(cls, device: torch.device, nbytes: int) -> torch.Tensor:
        key = (device.index, torch.cuda.current_stream(device).cuda_stream)
        buf = cls._bufs.get(key)
        if buf is None or buf.numel() < nbytes:
            buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
            cls._bufs[key] = buf
        return buf

    @classmethod
    def status_word(cls, device: torch.device) -> torch.Tensor:
        """One int32 per device that every call made through this module hands to the kernels: a kernel whose
        bounded wait runs out leaves DEVICE_TIMEOUT in it, and it stays there until device_status() reads it."""
        word = cls._status.get(device.index)
        if word is None:
            word = torch.zeros(1, dtype=torch.int32, device=device)
            cls._status[device.index] = word
        return word


def workspace_for(params: _cabi.SdpaParams, backward: bool, device: torch.device) -> torch.Tensor:
    lib = _cabi.load()
    need = ctypes.c_size_t(0)
    fn = lib.sdpa_b200_bwd_workspace_bytes if backward else lib.sdpa_b200_fwd_workspace_bytes
    _cabi.check(fn(ctypes.byref(params), ctypes.byref(need)), "workspace query")
    return _Workspace.get(device, need.value)


def _run(p: _cabi.SdpaParams, device: torch.device, backward: bool) -> None:
    # the library works on the current device and the stream it is given: make both the tensors' own
    lib = _cabi.load()
    with torch.cuda.device(device):
        p.device_status = _Workspace.status_word(device).data_ptr()
        ws = workspace_for(p, backward, device)
        fn = lib.sdpa_b200_bwd if backward else lib.sdpa_b200_fwd
        _cabi.check(fn(ctypes.byref(p), ws.data_ptr(), ws.numel(), _stream_ptr(device)),
                    "sdpa_b200_bwd" if backward else "sdpa_b200_fwd")


def _run_fwd(p: _cabi.SdpaParams, device: torch.device) -> None:
    _run(p, device, False)


def _run_bwd(p: _cabi.SdpaParams, device: torch.device) -> None:
    _run(p, device, True)


def device_status(device: Optional[torch.device] = None) -> int:
    """Synchronise the device's current stream and return what the kernels launched through this module since
    the last call of this function left in the device's status word: 0, or DEVICE_TIMEOUT when a bounded in-kernel
    wait ran out. The word is cleared on the way out."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    word = _Workspace.status_word(device)
    out = ctypes.c_int(0)
    with torch.cuda.device(device):
        _cabi.check(_cabi.load().sdpa_b200_read_device_status(word.data_ptr(), _stream_ptr(device), ctypes.byref(out)),
                    "read_device_status")
        if out.value != 0:
            word.zero_()
    return out.value


def check_device_status(device: Optional[torch.device] = None) -> None:
    """Raise when a kernel reported a time-out since the last check."""
    st = device_status(device)
    if st != 0:
        raise _cabi.SdpaError(st, "a kernel of this library gave up a bounded wait (DEVICE_TIMEOUT): its outputs are invalid")


def _empty_like_debug(q: torch.Tensor) -> torch.Tensor:
    return torch.empty((0,), dtype=q.dtype, device=q.device)


def _philox_placeholders(q: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    # dropout is 0: seed/offset are empty int64 tensors, as FlashAttention_internal.cpp:212-213
    e = torch.empty((0,), dtype=torch.int64, device=q.device)
    return e, e.clone()


# --------------------------------------------------------------------------------------
# dense [B, H, L, D]
# --------------------------------------------------------------------------------------
def _dense_params(query, key, value, out, lse, is_causal, scale, kernel=_cabi.KERNEL_AUTO,
                  num_splits=0) -> _cabi.SdpaParams:
    p = _cabi.SdpaParams()
    p.q, p.k, p.v = query.data_ptr(), key.data_ptr(), value.data_ptr()
    p.out, p.lse = out.data_ptr(), lse.data_ptr()
    p.batch, p.heads_q, p.heads_kv, p.head_dim = query.size(0), query.size(1), key.size(1), query.size(3)
    p.max_seqlen_q, p.max_seqlen_k = query.size(2), key.size(2)
    _set_strides_bhld(p, "q", query)
    _set_strides_bhld(p, "k", key)
    _set_strides_bhld(p, "v", value)
    _set_strides_bhld(p, "o", out)
    p.softmax_scale = scale
    p.dropout_p = 0.0
    p.is_causal = int(bool(is_causal))
    p.dtype = _cabi.DTYPE_F16 if query.dtype == torch.float16 else _cabi.DTYPE_BF16
    p.kernel = kernel
    p.num_splits = num_splits
    return p


def _set_bias(p: _cabi.SdpaParams, bias, dbias=None, bias_t=None) -> None:
    """bias / dbias: [B, H, Lq, Lk] views prepared by _prepare_bias / _new_bias_grad (unit key stride)."""
    if bias is None:
        return
    p.bias = bias.data_ptr()
    p.bias_batch_stride, p.bias_head_stride, p.bias_row_stride = bias.stride(0), bias.stride(1), bias.stride(2)
    if dbias is not None:
        p.dbias = dbias.data_ptr()
        p.dbias_batch_stride, p.dbias_head_stride, p.dbias_row_stride = dbias.stride(0), dbias.stride(1), dbias.stride(2)
    if bias_t is not None:
        p.bias_t = bias_t.data_ptr()
        p.bias_t_batch_stride, p.bias_t_head_stride, p.bias_t_row_stride = bias_t.stride(0), bias_t.stride(1), bias_t.stride(2)


def _transposed_bias(bias):
    """[B, H, Lk, Lq] view of a copy of ``bias`` (a [B, H, Lq, Lk] view from _prepare_bias) with keys and queries
    exchanged, for the backward: the dK/dV kernel's threads own keys and read consecutive queries. Broadcast
    batch / head dimensions stay broadcast; a bias that does not depend on the query needs no copy (None)."""
    if bias.stride(2) == 0:
        return None
    B, H, Lq, Lk = bias.shape
    nb, nh = (1 if bias.stride(0) == 0 else B), (1 if bias.stride(1) == 0 else H)
    lq8 = (Lq + 7) // 8 * 8
    buf = torch.empty((nb, nh, Lk, lq8), dtype=bias.dtype, device=bias.device)
    lib = _cabi.load()
    with torch.cuda.device(bias.device):
        _cabi.check(lib.sdpa_b200_transpose_bias(bias.data_ptr(), bias.stride(0), bias.stride(1), bias.stride(2), nb, nh, Lq, Lk,
                                                 buf.data_ptr(), lq8, _stream_ptr(bias.device)), "sdpa_b200_transpose_bias")
    return buf[..., :Lq].expand(B, H, Lk, Lq)


def _prepare_bias(attn_bias, query, key):
    """The additive bias as a [B, H, Lq, Lk] view the kernels can read: broadcast dimensions keep stride 0,
    rows start 16-byte aligned and are readable up to the next multiple of 8 keys. A bias that already has
    that layout is used in place; any other is copied once into rows padded to a multiple of 8."""
    B, H, Lq, _ = query.shape
    Lk = key.size(2)
    _check(attn_bias.dtype == query.dtype and attn_bias.device == query.device,
           "attn_bias must have the dtype and device of query")
    view = attn_bias.expand(B, H, Lq, Lk)
    ok = (view.stride(3) == 1 and Lk % 8 == 0 and view.data_ptr() % 16 == 0 and
          all(s % 8 == 0 for s in view.stride()[:3]))
    if ok:
        return view
    lk8 = (Lk + 7) // 8 * 8
    src = attn_bias.expand(*attn_bias.shape[:-1], Lk)
    buf = torch.zeros(*src.shape[:-1], lk8, dtype=query.dtype, device=query.device)
    buf[..., :Lk] = src
    return buf[..., :Lk].expand(B, H, Lq, Lk)


def _new_bias_grad(query, key):
    """Zero-filled [B, H, Lq, Lk] gradient buffer with rows padded to a multiple of 8 (the kernels skip what the
    causal mask hides)."""
    B, H, Lq, _ = query.shape
    Lk = key.size(2)
    return torch.zeros((B, H, Lq, (Lk + 7) // 8 * 8), dtype=query.dtype, device=query.device)[..., :Lk]


def _dense_forward(query, key, value, is_causal, scale, allow_gqa, kernel=_cabi.KERNEL_AUTO, num_splits=0, keep=None,
                   bias=None, sm_margin=0):
    # attention.cpp:70-100; `keep`: dropout.KeepMasks of this call, or None; `bias`: from _prepare_bias, or None
    _check(query.dim() == 4 and key.dim() == 4 and value.dim() == 4,
           "query, key and value must be 4-dimensional [batch, heads, seq_len, head_dim]")
    _check(query.size(0) == key.size(0) == value.size(0), "query, key and value must have the same batch size")
    _check(key.size(2) == value.size(2), "Key and Value must have the same sequence length")
    if allow_gqa:
        _check(key.size(1) == value.size(1) and query.size(1) % key.size(1) == 0,
               "Number of heads in key/value must divide number of heads in query")
    else:
        _check(query.size(1) == key.size(1) == value.size(1),
               "query, key and value must have the same number of heads")
    _check(query.size(3) == key.size(3) == value.size(3), "query, key and value must have the same head_dim")
    _check_inputs(query, key, value)
    B, H, Lq, D = query.shape
    # the reference returns a [B,H,L,D] view of a [B,L,H,D] buffer (attention.cpp:146-148)
    out = torch.empty((B, Lq, H, D), dtype=query.dtype, device=query.device).transpose(1, 2)
    lse = torch.empty((B, H, Lq), dtype=torch.float32, device=query.device)
    p = _dense_params(query, key, value, out, lse, is_causal, scale, kernel, num_splits)
    if keep is not None:
        p.dropout_p = keep.dropout_p
        p.keep_rows, p.keep_cols = keep.rows.data_ptr(), keep.cols.data_ptr()
    _set_bias(p, bias)
    p.sm_margin = int(sm_margin)
    _run_fwd(p, query.device)
    return out, lse


def _scaled_dot_product_flash_attention(query, key, value, dropout_p: float = 0.0, is_causal: bool = False,
                                        return_debug_mask: bool = False, *, scale: Optional[float] = None):
    """(output, logsumexp, cum_seq_q, cum_seq_k, max_q, max_k, philox_seed, philox_offset, debug_attn_mask).

    output is [B,H,Lq,D] bf16, logsumexp [B,H,ceil16(Lq)] fp32 (natural log, scale included; columns from Lq on
    are padding).
    """
    _check(0.0 <= dropout_p < 1.0, "dropout_p must be inside [0, 1)")
    _check(query.dim() == 4 and key.dim() == 4 and value.dim() == 4,
           "query, key and value must be 4-dimensional [batch, heads, seq_len, head_dim]")
    B, H, Lq, _ = query.shape
    Lk = key.size(2)
    keep = None
    seed, offset = _philox_placeholders(query)
    debug = _empty_like_debug(query)
    if dropout_p > 0.0:
        # With dropout the operator returns the Philox pair that fixes the pattern (FlashAttention_internal.cpp:
        # 190-214), as CPU int64 scalars, and on request the pattern itself (:141-146): > 0 where a pair was kept.
        s, o = dropout.draw_seed_and_offset(query.device, B * H * Lq * Lk)
        keep = dropout.dense_masks(s, o, dropout_p, B, H, Lq, Lk, query.device, is_causal, forward=True)
        seed, offset = torch.tensor(s, dtype=torch.int64), torch.tensor(o, dtype=torch.int64)
        if return_debug_mask:
            debug = keep.dense().to(query.dtype)
    out, lse = _dense_forward(query, key, value, is_causal, calculate_scale(query, scale), allow_gqa=False, keep=keep)
    if Lq % 16 != 0:
        # the reference hands the logsumexp back with its last dimension rounded up to 16
        # (FlashAttention_internal.cpp:261-265); the padding holds zeros and the backward operator cuts it off (:374-375)
        lse = torch.nn.functional.pad(lse, (0, (Lq + 15) // 16 * 16 - Lq))
    # attention.cpp:109-119; kept for callers that pass them on to the backward op
    cum_q = torch.arange(0, (B + 1) * Lq, Lq, dtype=torch.int32, device=query.device)
    cum_k = torch.arange(0, (B + 1) * Lk, Lk, dtype=torch.int32, device=query.device)
    return out, lse, cum_q, cum_k, Lq, Lk, seed, offset, debug


def _deterministic(flag: Optional[bool]) -> int:
    """The backward's `deterministic` switch: an explicit choice, else torch's global setting."""
    return int(torch.are_deterministic_algorithms_enabled() if flag is None else bool(flag))


def _dense_backward(grad_out, query, key, value, out, logsumexp, is_causal, scale, keep=None, bias=None, dbias=None,
                    bias_t=None, deterministic: Optional[bool] = None):
    # bias_t: a transposed copy of the bias (see _transposed_bias) kept by the caller; made here when missing
    # deterministic: True = the kernels with a fixed summation order; None = torch.are_deterministic_algorithms_enabled()
    _check_inputs(grad_out, query, key, value, out)
    _check(logsumexp.dtype == torch.float32 and logsumexp.is_contiguous(), "logsumexp must be contiguous fp32")
    B, H, Lq, D = query.shape
    _check(tuple(logsumexp.shape) == (B, H, Lq), "logsumexp must be [batch, heads, seqlen_q]")
    dq = torch.empty((B, Lq, H, D), dtype=query.dtype, device=query.device).transpose(1, 2)
    dk = torch.empty((B, key.size(2), key.size(1), D), dtype=key.dtype, device=key.device).transpose(1, 2)
    dv = torch.empty((B, key.size(2), key.size(1), D), dtype=key.dtype, device=key.device).transpose(1, 2)
    p = _dense_params(query, key, value, out, logsumexp, is_causal, scale)
    p.dout, p.dq, p.dk, p.dv = grad_out.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    _set_strides_bhld(p, "do", grad_out)
    _set_strides_bhld(p, "dq", dq)
    _set_strides_bhld(p, "dk", dk)
    _set_strides_bhld(p, "dv", dv)
    if keep is not None:
        p.dropout_p = keep.dropout_p
        p.keep_rows, p.keep_cols = keep.rows.data_ptr(), keep.cols.data_ptr()
    if bias_t is False:
        bias_t = None  # the caller wants the strided reads (tests compare the two paths)
    elif bias is not None and bias_t is None:
        bias_t = _transposed_bias(bias)  # one HBM pass; the dK/dV kernel then reads the bias 16 bytes at a time
    _set_bias(p, bias, dbias, bias_t)
    p.deterministic = _deterministic(deterministic)
    _run_bwd(p, query.device)
    return dq, dk, dv


def _scaled_dot_product_flash_attention_backward(grad_out, query, key, value, out, logsumexp, cum_seq_q, cum_seq_k,
                                                 max_q, max_k, dropout_p, is_causal, philox_seed, philox_offset,
                                                 *, scale: Optional[float] = None):
    """(grad_q, grad_k, grad_v), each shaped like its input (attention.cpp:205-297). With dropout the pattern
    of the forward call is drawn again from ``philox_seed`` / ``philox_offset``."""
    _check(0.0 <= dropout_p < 1.0, "dropout_p must be inside [0, 1)")
    if grad_out.stride(-1) != 1:
        grad_out = grad_out.contiguous()
    keep = None
    if dropout_p > 0.0:
        _check(philox_seed.numel() == 1 and philox_offset.numel() == 1,
               "dropout_p > 0 needs the philox_seed and philox_offset the forward operator returned")
        B, H, Lq, _ = query.shape
        keep = dropout.dense_masks(int(philox_seed), int(philox_offset), dropout_p, B, H, Lq, key.size(2), query.device,
                                   is_causal, forward=False)
    if logsumexp.size(-1) != query.size(2):
        logsumexp = logsumexp[..., :query.size(2)].contiguous()
    return _dense_backward(grad_out, query, key, value, out, logsumexp, is_causal, calculate_scale(query, scale), keep=keep)


# --------------------------------------------------------------------------------------
# memory-efficient operator surface
# --------------------------------------------------------------------------------------
def _scaled_dot_product_efficient_attention(query, key, value, attn_bias, compute_log_sumexp: bool,
                                            dropout_p: float = 0.0, is_causal: bool = False, *,
                                            scale: Optional[float] = None):
    """(output, log_sumexp, philox_seed, philox_offset), attention.cpp:350-391.

    The reference runs this operator on the same device kernel as the flash operator; what differs at
    this level is the additive ``attn_bias`` (anything that broadcasts to [B, H, Lq, Lk], in the dtype of
    query) and the causal convention: ``CausalFromTopLeft`` (sdp_utils.h:32-37, attention.cpp:369-371)
    instead of the flash operator's bottom-right alignment. With Lq == Lk the two coincide; otherwise
    the top-left mask is rebuilt from what the kernels offer: keys past Lq are invisible to every row
    (Lq < Lk), and rows past Lk see every key (Lq > Lk).
    ``log_sumexp`` is [B,H,Lq] fp32, or empty when ``compute_log_sumexp`` is false. With dropout the Philox pair
    comes back as two CPU int64 scalars.
    """
    _check(0.0 <= dropout_p < 1.0, "dropout_p must be inside [0, 1)")
    _check(query.dim() == 4 and key.dim() == 4, "query, key and value must be 4-dimensional [batch, heads, seq_len, head_dim]")
    sc = calculate_scale(query, scale)
    Lq, Lk = query.size(2), key.size(2)
    bias = None if attn_bias is None else _prepare_bias(attn_bias, query, key)
    sl = (lambda t, *idx: None if t is None else t[idx])  # slices of an optional tensor
    seed, offset = _philox_placeholders(query)
    keep_for = lambda lq, lk, causal, part: None
    if dropout_p > 0.0:
        s0, o0 = dropout.draw_seed_and_offset(query.device, query.size(0) * query.size(1) * Lq * Lk)
        seed, offset = torch.tensor(s0, dtype=torch.int64), torch.tensor(o0, dtype=torch.int64)
        keep_for = _keep_factory(s0, o0, dropout_p, query, True)
    if not is_causal or Lq == Lk:
        out, lse = _dense_forward(query, key, value, is_causal, sc, allow_gqa=False, bias=bias, keep=keep_for(Lq, Lk, is_causal, 0))
    elif Lq < Lk:
        out, lse = _dense_forward(query, key[:, :, :Lq], value[:, :, :Lq], True, sc, allow_gqa=False,
                                  bias=sl(bias, Ellipsis, slice(0, Lq)), keep=keep_for(Lq, Lq, True, 0))
    else:
        o1, l1 = _dense_forward(query[:, :, :Lk], key, value, True, sc, allow_gqa=False,
                                bias=sl(bias, slice(None), slice(None), slice(0, Lk)), keep=keep_for(Lk, Lk, True, 0))
        o2, l2 = _dense_forward(query[:, :, Lk:], key, value, False, sc, allow_gqa=False,
                                bias=sl(bias, slice(None), slice(None), slice(Lk, None)), keep=keep_for(Lq - Lk, Lk, False, 1))
        out = torch.cat([o1.transpose(1, 2), o2.transpose(1, 2)], dim=1).transpose(1, 2)
        lse = torch.cat([l1, l2], dim=2)
    if not compute_log_sumexp:
        lse = lse.new_empty((query.size(0), query.size(1), 0))
    return out, lse, seed, offset


def _keep_factory(seed: int, offset: int, dropout_p: float, query, forward: bool):
    """Keep-masks for the kernel calls one memory-efficient operator call is made of: the same Philox pair, the
    second call (rows past Lk of a top-left causal mask) on a stream of its own (bit 62 of the offset)."""
    B, H = query.size(0), query.size(1)
    return lambda lq, lk, causal, part: dropout.dense_masks(seed, offset ^ (part << 62), dropout_p, B, H, lq, lk, query.device,
                                                            causal, forward=forward)


def _philox_ints(philox_seed, philox_offset) -> Tuple[int, int]:
    _check(philox_seed.numel() == 1 and philox_offset.numel() == 1,
           "dropout_p > 0 needs the philox_seed and philox_offset the forward operator returned")
    return int(philox_seed), int(philox_offset)


def _scaled_dot_product_efficient_attention_backward(grad_out, query, key, value, attn_bias, out, logsumexp,
                                                     philox_seed, philox_offset, dropout_p: float,
                                                     grad_input_mask, is_causal: bool = False, *,
                                                     scale: Optional[float] = None):
    """(grad_q, grad_k, grad_v, grad_bias), attention.cpp:510-600. Needs the log_sumexp of a forward call with
    ``compute_log_sumexp=True``. grad_bias has the shape of ``attn_bias`` (the [B, H, Lq, Lk] gradient the kernel
    writes, summed over the dimensions the bias broadcasts along) when ``grad_input_mask[3]`` asks for it, else it
    is an empty tensor."""
    has_bias = attn_bias is not None and attn_bias.numel() > 0
    _check(0.0 <= dropout_p < 1.0, "dropout_p must be inside [0, 1)")
    _check(logsumexp.size(-1) == query.size(2), "log_sumexp is empty: run the forward with compute_log_sumexp=True")
    sc = calculate_scale(query, scale)
    if grad_out.stride(-1) != 1:
        grad_out = grad_out.contiguous()
    Lq, Lk = query.size(2), key.size(2)
    bias = _prepare_bias(attn_bias, query, key) if has_bias else None
    want_dbias = has_bias and len(grad_input_mask) > 3 and bool(grad_input_mask[3])
    dbias = _new_bias_grad(query, key) if want_dbias else None
    sl = (lambda t, *idx: None if t is None else t[idx])

    def finish(dq, dk, dv):
        if dbias is None:
            return dq, dk, dv, query.new_empty((0,))
        return dq, dk, dv, dbias.sum_to_size(attn_bias.shape)

    keep_for = lambda lq, lk, causal, part: None
    if dropout_p > 0.0:
        _check(philox_seed.numel() == 1 and philox_offset.numel() == 1,
               "dropout_p > 0 needs the philox_seed and philox_offset the forward operator returned")
        keep_for = _keep_factory(int(philox_seed), int(philox_offset), dropout_p, query, False)
    if not is_causal or Lq == Lk:
        dq, dk, dv = _dense_backward(grad_out, query, key, value, out, logsumexp, is_causal, sc, bias=bias, dbias=dbias,
                                     keep=keep_for(Lq, Lk, is_causal, 0))
    elif Lq < Lk:
        cut = (Ellipsis, slice(0, Lq))
        dq, dk_a, dv_a = _dense_backward(grad_out, query, key[:, :, :Lq], value[:, :, :Lq], out, logsumexp, True, sc,
                                         bias=sl(bias, *cut), dbias=sl(dbias, *cut), keep=keep_for(Lq, Lq, True, 0))
        dk, dv = torch.zeros_like(key), torch.zeros_like(value)
        dk[:, :, :Lq] = dk_a
        dv[:, :, :Lq] = dv_a
    else:
        top, rest = (slice(None), slice(None), slice(0, Lk)), (slice(None), slice(None), slice(Lk, None))
        l1, l2 = logsumexp[:, :, :Lk].contiguous(), logsumexp[:, :, Lk:].contiguous()
        dq1, dk1, dv1 = _dense_backward(grad_out[:, :, :Lk], query[:, :, :Lk], key, value, out[:, :, :Lk], l1, True, sc,
                                        bias=sl(bias, *top), dbias=sl(dbias, *top), keep=keep_for(Lk, Lk, True, 0))
        dq2, dk2, dv2 = _dense_backward(grad_out[:, :, Lk:], query[:, :, Lk:], key, value, out[:, :, Lk:], l2, False, sc,
                                        bias=sl(bias, *rest), dbias=sl(dbias, *rest), keep=keep_for(Lq - Lk, Lk, False, 1))
        dq = torch.cat([dq1.transpose(1, 2), dq2.transpose(1, 2)], dim=1).transpose(1, 2)
        dk = (dk1.float() + dk2.float()).to(key.dtype)
        dv = (dv1.float() + dv2.float()).to(value.dtype)
    return finish(dq, dk, dv)


# --------------------------------------------------------------------------------------
# packed varlen [total, H, D] + int32 cu_seqlens
# --------------------------------------------------------------------------------------
def _varlen_params(query, key, value, out, lse, cu_q, cu_k, max_q, max_k, is_causal, scale) -> _cabi.SdpaParams:
    p = _cabi.SdpaParams()
    p.q, p.k, p.v = query.data_ptr(), key.data_ptr(), value.data_ptr()
    p.out, p.lse = out.data_ptr(), lse.data_ptr()
    p.cu_seqlens_q, p.cu_seqlens_k = cu_q.data_ptr(), cu_k.data_ptr()
    p.batch = cu_q.numel() - 1
    p.heads_q, p.heads_kv, p.head_dim = query.size(1), key.size(1), query.size(2)
    p.max_seqlen_q, p.max_seqlen_k = int(max_q), int(max_k)
    p.total_q, p.total_k = query.size(0), key.size(0)
    _set_strides_thd(p, "q", query)
    _set_strides_thd(p, "k", key)
    _set_strides_thd(p, "v", value)
    _set_strides_thd(p, "o", out)
    p.softmax_scale = scale
    p.dropout_p = 0.0
    p.is_causal = int(bool(is_causal))
    p.dtype = _cabi.DTYPE_F16 if query.dtype == torch.float16 else _cabi.DTYPE_BF16
    p.kernel = _cabi.KERNEL_PREFILL
    return p


def _check_varlen(query, key, value, cu_q, cu_k):
    # FlashAttention_internal.cpp:81-84, 112-127
    _check(query.dim() == 3 and key.dim() == 3 and value.dim() == 3,
           "varlen query, key and value must be packed [total_tokens, heads, head_dim]")
    _check(cu_q.dtype == torch.int32, "cu_seqlens_q must have dtype int32")
    _check(cu_k.dtype == torch.int32, "cu_seqlens_k must have dtype int32")
    _check(cu_q.is_cuda and cu_k.is_cuda, "cu_seqlens must be on the device")
    _check(cu_q.is_contiguous() and cu_k.is_contiguous(), "cu_seqlens must be contiguous")
    _check(cu_q.numel() == cu_k.numel() and cu_q.numel() >= 2, "cu_seqlens_q and cu_seqlens_k must have batch+1 entries")
    _check(key.size(1) == value.size(1) and query.size(1) % key.size(1) == 0,
           "Number of heads in key/value must divide number of heads in query")
    _check(query.size(2) == key.size(2) == value.size(2), "query, key and value must have the same head_dim")
    _check(key.size(0) == value.size(0), "Key and Value must have the same number of tokens")
    _check_inputs(query, key, value)


def _varlen_forward(query, key, value, cu_q, cu_k, max_q, max_k, is_causal, scale, keep=None, bias=None):
    """Packed forward: (out [total_q, Hq, D], lse [Hq, total_q]). `keep`: dropout.KeepMasksVarlen or None; `bias`: a
    [B, Hq, max_q, max_k] view from _prepare_bias or None (sequence b reads bias[b] by positions inside the sequence)."""
    _check_varlen(query, key, value, cu_q, cu_k)
    out = torch.empty_like(query, memory_format=torch.contiguous_format)
    lse = torch.empty((query.size(1), query.size(0)), dtype=torch.float32, device=query.device)
    p = _varlen_params(query, key, value, out, lse, cu_q, cu_k, max_q, max_k, is_causal, scale)
    if keep is not None:
        p.dropout_p = keep.dropout_p
        p.keep_rows, p.keep_cols = keep.rows.data_ptr(), keep.cols.data_ptr()
    _set_bias(p, bias)
    _run_fwd(p, query.device)
    return out, lse


def _varlen_backward(grad_out, query, key, value, out, logsumexp, cu_q, cu_k, max_q, max_k, is_causal, scale, keep=None,
                     bias=None, dbias=None, deterministic: Optional[bool] = None):
    _check_varlen(query, key, value, cu_q, cu_k)
    if grad_out.stride(-1) != 1:
        grad_out = grad_out.contiguous()
    _check_inputs(grad_out, out)
    _check(logsumexp.dtype == torch.float32 and logsumexp.is_contiguous()
           and tuple(logsumexp.shape) == (query.size(1), query.size(0)),
           "logsumexp must be contiguous fp32 [heads_q, total_q]")
    dq = torch.empty_like(query, memory_format=torch.contiguous_format)
    dk = torch.empty_like(key, memory_format=torch.contiguous_format)
    dv = torch.empty_like(value, memory_format=torch.contiguous_format)
    p = _varlen_params(query, key, value, out, logsumexp, cu_q, cu_k, max_q, max_k, is_causal, scale)
    p.dout, p.dq, p.dk, p.dv = grad_out.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    _set_strides_thd(p, "do", grad_out)
    _set_strides_thd(p, "dq", dq)
    _set_strides_thd(p, "dk", dk)
    _set_strides_thd(p, "dv", dv)
    if keep is not None:
        p.dropout_p = keep.dropout_p
        p.keep_rows, p.keep_cols = keep.rows.data_ptr(), keep.cols.data_ptr()
    _set_bias(p, bias, dbias, None if bias is None else _transposed_bias(bias))
    p.deterministic = _deterministic(deterministic)
    _run_bwd(p, query.device)
    return dq, dk, dv


def _flash_attention_forward(query, key, value, cum_seq_q, cum_seq_k, max_q: int, max_k: int, dropout_p: float,
                             is_causal: bool, return_debug_mask: bool, *, scale: Optional[float] = None):
    """(output, softmax_logsumexp, philox_seed, philox_offset, debug_attn_mask).

    output is [total_q, Hq, D]; softmax_logsumexp is [Hq, total_q] fp32, the buffer
    mha_varlen_fwd allocates (FlashAttention_internal.cpp:129). The reference then views it
    as [Hq, B, max_q] (:261-265), which only exists for equal-length batches; ragged batches
    keep the packed layout here.
    """
    _check(0.0 <= dropout_p < 1.0, "dropout_p must be inside [0, 1)")
    _check_varlen(query, key, value, cum_seq_q, cum_seq_k)
    seed, offset = _philox_placeholders(query)
    debug = _empty_like_debug(query)
    keep = None
    if dropout_p > 0.0:
        # the Philox pair as two CPU int64 scalars; on request the pattern as [B, Hq, max_q, max_k], > 0 = kept
        s, o = dropout.draw_seed_and_offset(query.device, (cum_seq_q.numel() - 1) * query.size(1) * int(max_q) * int(max_k))
        keep = dropout.packed_masks(s, o, dropout_p, query.size(1), cum_seq_q, cum_seq_k, query.size(0), key.size(0),
                                    int(max_q), int(max_k), is_causal, forward=True)
        seed, offset = torch.tensor(s, dtype=torch.int64), torch.tensor(o, dtype=torch.int64)
        if return_debug_mask:
            debug = keep.dense().to(query.dtype)
    out, lse = _varlen_forward(query, key, value, cum_seq_q, cum_seq_k, max_q, max_k, is_causal, calculate_scale(query, scale),
                               keep=keep)
    return out, lse, seed, offset, debug


def _flash_attention_backward(grad_out, query, key, value, out, logsumexp, cum_seq_q, cum_seq_k, max_q: int,
                              max_k: int, dropout_p: float, is_causal: bool, philox_seed, philox_offset,
                              *, scale: Optional[float] = None):
    """(dq, dk, dv) for packed varlen tensors. dk/dv have Hkv heads: the GQA group is reduced
    inside the kernel (the reference's shape check at FlashAttention_internal.cpp:363-364
    cannot pass for Hq != Hkv; here it can)."""
    _check(0.0 <= dropout_p < 1.0, "dropout_p must be inside [0, 1)")
    _check_varlen(query, key, value, cum_seq_q, cum_seq_k)
    keep = None
    if dropout_p > 0.0:
        s, o = _philox_ints(philox_seed, philox_offset)
        keep = dropout.packed_masks(s, o, dropout_p, query.size(1), cum_seq_q, cum_seq_k, query.size(0), key.size(0),
                                    int(max_q), int(max_k), is_causal, forward=False)
    return _varlen_backward(grad_out, query, key, value, out, logsumexp, cum_seq_q, cum_seq_k, max_q, max_k, is_causal,
                            calculate_scale(query, scale), keep=keep)


# --------------------------------------------------------------------------------------
# memory-efficient operators on [B, L, H, D] tensors
# --------------------------------------------------------------------------------------
# sdp::CustomMaskType (sdp_utils.h:32-37)
NO_CUSTOM_MASK, CAUSAL_FROM_TOP_LEFT, CAUSAL_FROM_BOTTOM_RIGHT = 0, 1, 2


def _efficient_attention_forward(query, key, value, bias, cu_seqlens_q, cu_seqlens_k, max_seqlen_q: Optional[int],
                                 dropout_p: float, custom_mask_type: int, compute_log_sumexp: bool = False, *,
                                 scale: Optional[float] = None, causal_diagonal=None, seqlen_k=None):
    """(output, logsumexp, philox_seed, philox_offset), attention.cpp:393-507.

    query is [B, Lq, H, D], key / value [B, Lk, H, D] (sequence before heads, unlike the sdp operators).
    output comes back as the reference returns it: the [B, Lq, H, D] buffer viewed as [B, H, Lq, D]
    (:503-506). logsumexp is [H, B*Lq] fp32 (mem_eff_fwd, FlashAttention_internal.cpp:603), empty unless
    asked for. ``bias`` is [B, H, Lq, Lk] or anything that broadcasts to it; with dropout the Philox pair comes
    back as two CPU int64 scalars. With cu_seqlens (int32 [B+1], offsets into the flattened B*L token axis,
    :435-470) the packed kernels run: sequence b reads bias[b] by positions counted from its own start, and the
    causal mask is bottom-right aligned, so ``CausalFromTopLeft`` is taken there only when both offset tensors are
    equal (the two alignments then coincide).
    """
    _check(query.dim() == 4 and key.dim() == 4 and value.dim() == 4, "query, key and value must be [B, L, H, D]")
    _check(query.size(0) == key.size(0) == value.size(0), "batch sizes differ")
    _check(key.size(1) == value.size(1), "key and value lengths differ")
    _check(query.size(2) == key.size(2) == value.size(2), "numbers of heads differ")
    _check(query.size(3) == key.size(3) == value.size(3), "head dims differ")
    _check(0.0 <= dropout_p < 1.0, "dropout_p must be inside [0, 1)")
    _check(causal_diagonal is None and seqlen_k is None, "causal_diagonal and seqlen_k are not supported")
    _check(custom_mask_type in (NO_CUSTOM_MASK, CAUSAL_FROM_TOP_LEFT, CAUSAL_FROM_BOTTOM_RIGHT),
           f"unknown custom_mask_type {custom_mask_type}")
    _check((cu_seqlens_q is None) == (cu_seqlens_k is None), "cu_seqlens_q and cu_seqlens_k must be given together")
    B, Lq, H, D = query.shape
    Lk = key.size(1)
    sc = calculate_scale(query, scale)
    seed, offset = _philox_placeholders(query)
    q_t, k_t, v_t = query.transpose(1, 2), key.transpose(1, 2), value.transpose(1, 2)
    if cu_seqlens_q is None:
        if custom_mask_type == CAUSAL_FROM_TOP_LEFT:
            out, lse, seed, offset = _scaled_dot_product_efficient_attention(q_t, k_t, v_t, bias, True, dropout_p, True, scale=sc)
        else:
            causal = custom_mask_type == CAUSAL_FROM_BOTTOM_RIGHT
            keep = None
            if dropout_p > 0.0:
                s, o = dropout.draw_seed_and_offset(query.device, B * H * Lq * Lk)
                seed, offset = torch.tensor(s, dtype=torch.int64), torch.tensor(o, dtype=torch.int64)
                keep = dropout.dense_masks(s, o, dropout_p, B, H, Lq, Lk, query.device, causal, forward=True)
            out, lse = _dense_forward(q_t, k_t, v_t, causal, sc, allow_gqa=False, keep=keep,
                                      bias=None if bias is None else _prepare_bias(bias, q_t, k_t))
        lse = lse.permute(1, 0, 2).reshape(H, B * Lq)
    else:
        _check(cu_seqlens_q.dtype == torch.int32 and cu_seqlens_k.dtype == torch.int32, "cu_seqlens must have dtype int32")
        _check(cu_seqlens_q.numel() == B + 1 and cu_seqlens_k.numel() == B + 1, "cu_seqlens must have batch + 1 entries")
        causal = custom_mask_type != NO_CUSTOM_MASK
        if custom_mask_type == CAUSAL_FROM_TOP_LEFT:
            _check(cu_seqlens_q is cu_seqlens_k or torch.equal(cu_seqlens_q, cu_seqlens_k),
                   "CausalFromTopLeft with cu_seqlens needs equal query and key lengths in this library")
        max_q = Lq if max_seqlen_q is None else int(max_seqlen_q)
        cu_q, cu_k = cu_seqlens_q.contiguous(), cu_seqlens_k.contiguous()
        keep = None
        if dropout_p > 0.0:
            s, o = dropout.draw_seed_and_offset(query.device, B * H * max_q * Lk)
            seed, offset = torch.tensor(s, dtype=torch.int64), torch.tensor(o, dtype=torch.int64)
            keep = dropout.packed_masks(s, o, dropout_p, H, cu_q, cu_k, B * Lq, B * Lk, max_q, Lk, causal, forward=True)
        out, lse = _varlen_forward(query.reshape(B * Lq, H, D), key.reshape(B * Lk, H, D), value.reshape(B * Lk, H, D), cu_q,
                                   cu_k, max_q, Lk, causal, sc, keep=keep,
                                   bias=None if bias is None else _prepare_bias(bias, q_t, k_t))
        out = out.view(B, Lq, H, D).transpose(1, 2)
    if not compute_log_sumexp:
        lse = lse.new_empty((0,))
    return out, lse, seed, offset


def _efficient_attention_backward(grad_out_, query, key, value, bias, out, cu_seqlens_q, cu_seqlens_k, max_seqlen_k: int,
                                  max_seqlen_q: int, logsumexp, dropout_p: float, philox_seed, philox_offset,
                                  custom_mask_type: int, bias_requires_grad: bool, *, scale: Optional[float] = None,
                                  num_splits_key: Optional[int] = None):
    """(grad_q [B,Lq,H,D], grad_k, grad_v [B,Lk,H,D], grad_bias), attention.cpp:579-727, for a forward call
    ``out`` and ``grad_out_`` are [B, Lq, H, D] (any strides with unit head-dim stride); ``logsumexp`` is the
    [H, B*Lq] tensor of the forward. grad_bias is shaped like ``bias`` when ``bias_requires_grad``, else empty.
    With ``dropout_p`` the pattern of the forward call is drawn again from ``philox_seed`` / ``philox_offset``."""
    _check(0.0 <= dropout_p < 1.0, "dropout_p must be inside [0, 1)")
    _check(query.dim() == 4 and grad_out_.dim() == 4 and out.dim() == 4, "tensors must be [B, L, H, D]")
    _check((cu_seqlens_q is None) == (cu_seqlens_k is None), "cu_seqlens_q and cu_seqlens_k must be given together")
    B, Lq, H, D = query.shape
    Lk = key.size(1)
    _check(tuple(logsumexp.shape) == (H, B * Lq), "logsumexp must be [heads, batch*seqlen_q]: run the forward with "
                                                  "compute_log_sumexp=True")
    sc = calculate_scale(query, scale)
    empty_bias_grad = query.new_empty((0,))
    t = lambda x: x.transpose(1, 2)
    want_dbias = bias is not None and bool(bias_requires_grad)
    if cu_seqlens_q is None:
        lse = logsumexp.view(H, B, Lq).permute(1, 0, 2).contiguous()
        if custom_mask_type == CAUSAL_FROM_TOP_LEFT:
            dq, dk, dv, db = _scaled_dot_product_efficient_attention_backward(
                t(grad_out_), t(query), t(key), t(value), bias, t(out), lse, philox_seed, philox_offset, dropout_p,
                [True, True, True, want_dbias], True, scale=sc)
        else:
            causal = custom_mask_type == CAUSAL_FROM_BOTTOM_RIGHT
            go = t(grad_out_)
            if go.stride(-1) != 1:
                go = go.contiguous()
            b4 = None if bias is None else _prepare_bias(bias, t(query), t(key))
            dfull = _new_bias_grad(t(query), t(key)) if want_dbias else None
            keep = None
            if dropout_p > 0.0:
                s, o = _philox_ints(philox_seed, philox_offset)
                keep = dropout.dense_masks(s, o, dropout_p, B, H, Lq, Lk, query.device, causal, forward=False)
            dq, dk, dv = _dense_backward(go, t(query), t(key), t(value), t(out), lse, causal, sc, bias=b4, dbias=dfull,
                                         keep=keep)
            db = dfull.sum_to_size(bias.shape) if want_dbias else empty_bias_grad
        return t(dq), t(dk), t(dv), db
    causal = custom_mask_type != NO_CUSTOM_MASK
    if custom_mask_type == CAUSAL_FROM_TOP_LEFT:
        _check(cu_seqlens_q is cu_seqlens_k or torch.equal(cu_seqlens_q, cu_seqlens_k),
               "CausalFromTopLeft with cu_seqlens needs equal query and key lengths in this library")
    cu_q, cu_k = cu_seqlens_q.contiguous(), cu_seqlens_k.contiguous()
    keep = None
    if dropout_p > 0.0:
        s, o = _philox_ints(philox_seed, philox_offset)
        keep = dropout.packed_masks(s, o, dropout_p, H, cu_q, cu_k, B * Lq, B * Lk, int(max_seqlen_q), int(max_seqlen_k), causal,
                                    forward=False)
    b4 = None if bias is None else _prepare_bias(bias, t(query), t(key))
    dfull = _new_bias_grad(t(query), t(key)) if want_dbias else None
    dq, dk, dv = _varlen_backward(grad_out_.reshape(B * Lq, H, D), query.reshape(B * Lq, H, D), key.reshape(B * Lk, H, D),
                                  value.reshape(B * Lk, H, D), out.reshape(B * Lq, H, D), logsumexp.contiguous(), cu_q, cu_k,
                                  int(max_seqlen_q), int(max_seqlen_k), causal, sc, keep=keep, bias=b4, dbias=dfull)
    db = dfull.sum_to_size(bias.shape) if want_dbias else empty_bias_grad
    return dq.view(B, Lq, H, D), dk.view(B, Lk, H, D), dv.view(B, Lk, H, D), db


def decode_attention(query, key_cache, value_cache, *, scale: Optional[float] = None, num_splits: int = 0):
    """query [B,Hq,1,D], key/value cache [B,Hkv,Lkv,D] -> (output [B,Hq,1,D], logsumexp [B,Hq,1]).

    Split-KV streaming kernel; the key range is cut into ``num_splits`` pieces (0 = choose)."""
    _check(query.dim() == 4 and query.size(2) == 1, "decode_attention needs query of shape [B, Hq, 1, D]")
    out, lse = _dense_forward(query, key_cache, value_cache, False, calculate_scale(query, scale),
                              allow_gqa=True, kernel=_cabi.KERNEL_DECODE, num_splits=num_splits)
    return out, lse


def gqa_prefill(query, key, value, *, is_causal: bool = False, scale: Optional[float] = None, sm_margin: int = 0):
    """Dense [B,Hq,L,D] x [B,Hkv,L,D] prefill with head broadcast (the dense reference op
    refuses Hq != Hkv, attention.cpp:82-83; the kernel underneath does not). ``sm_margin`` SMs are left free
    for a kernel that runs beside this one on another stream (a collective, for example)."""
    return _dense_forward(query, key, value, is_causal, calculate_scale(query, scale), allow_gqa=True,
                          kernel=_cabi.KERNEL_PREFILL, sm_margin=sm_margin)
