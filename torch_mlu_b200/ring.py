"""Ring / context-parallel prefill for sequences too long for one GPU's share of the work.

Every rank owns a contiguous slice of the sequence: its queries stay put, the key/value slices
travel around the ring (``batch_isend_irecv`` over NCCL: each hop lands in this GPU's own memory
before any kernel reads it). At every hop the local forward kernel produces a partial
(out, logsumexp) for (local queries x visiting keys) and ``merge_partial`` folds it into an fp32
accumulator by the logsumexp rule. Causal masking falls out of the slice order: a visiting slice
from an earlier rank is fully visible, the rank's own slice is the usual lower triangle, slices
from later ranks are skipped (but still forwarded).

The reference has no such path (its attention is single-device; P2P lives in
ProcessGroupCNCL::send/recv, process_group_cncl.cpp:2526-2552).
"""
from __future__ import annotations

import ctypes
import functools
from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

from . import _cabi


def merge_partial(o_acc: torch.Tensor, lse_acc: torch.Tensor, o_part: torch.Tensor, lse_part: torch.Tensor) -> None:
    """In-place logsumexp fold of a bf16 / f16 partial [B,H,L,D] (any strides) into the fp32
    accumulator (contiguous [B,H,L,D], lse [B,H,L]). CUDA only."""
    assert o_acc.is_cuda and o_acc.dtype == torch.float32 and o_acc.is_contiguous()
    assert lse_acc.dtype == torch.float32 and lse_acc.is_contiguous() and lse_part.is_contiguous()
    assert o_part.dtype in (torch.bfloat16, torch.float16) and o_part.stride(-1) == 1
    B, H, L, D = o_acc.shape
    lib = _cabi.load()
    with torch.cuda.device(o_acc.device):  # the library launches on the current device
        st = lib.sdpa_b200_merge_partial(o_acc.data_ptr(), lse_acc.data_ptr(), o_part.data_ptr(), lse_part.data_ptr(), B, H, L, D,
                                         _cabi.DTYPE_F16 if o_part.dtype == torch.float16 else _cabi.DTYPE_BF16,
                                         o_part.stride(0), o_part.stride(1), o_part.stride(2),
                                         torch.cuda.current_stream(o_acc.device).cuda_stream)
    _cabi.check(st, "sdpa_b200_merge_partial")


def merge_partial_reference(o_acc, lse_acc, o_part, lse_part) -> None:
    """The same fold in plain torch (host-side logic tests on CPU ranks)."""
    lp = torch.where(torch.isposinf(lse_part), torch.full_like(lse_part, float("-inf")), lse_part)
    new = torch.logaddexp(lse_acc, lp)
    wa = torch.where(torch.isneginf(new), torch.zeros_like(new), torch.exp(lse_acc - new))
    wp = torch.where(torch.isneginf(new), torch.zeros_like(new), torch.exp(lp - new))
    o_acc.copy_(torch.where(wa.unsqueeze(-1) == 0, torch.zeros_like(o_acc), o_acc * wa.unsqueeze(-1)) + o_part.float() * wp.unsqueeze(-1))
    lse_acc.copy_(new)


def zigzag_rows(rank: int, world: int, seqlen: int) -> Tuple[slice, slice]:
    """Row ranges of ``rank`` in the zig-zag layout: the sequence is cut into 2*world chunks and rank r
    owns chunks r and 2*world-1-r, so every rank holds the same share of a causal mask's work."""
    assert seqlen % (2 * world) == 0, "zig-zag layout needs seqlen divisible by 2*world"
    c = seqlen // (2 * world)
    return slice(rank * c, (rank + 1) * c), slice((2 * world - 1 - rank) * c, (2 * world - rank) * c)


def zigzag_take(x: torch.Tensor, rank: int, world: int, dim: int = 2) -> torch.Tensor:
    """The slice of ``x`` (full sequence along ``dim``) that ``rank`` owns in the zig-zag layout."""
    lo, hi = zigzag_rows(rank, world, x.size(dim))
    idx = [slice(None)] * x.dim()
    idx[dim] = lo
    first = x[tuple(idx)]
    idx[dim] = hi
    return torch.cat([first, x[tuple(idx)]], dim=dim)


def ring_prefill(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, is_causal: bool, scale: Optional[float] = None,
                 group=None, attention_fn: Optional[Callable] = None, merge_fn: Optional[Callable] = None,
                 layout: str = "contiguous", exchange: bool = True, sm_margin: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """q [B,Hq,Ls,D], k/v [B,Hkv,Ls,D]: this rank's slice of the sequence.
    ``layout="contiguous"``: rank r owns rows [r*Ls, (r+1)*Ls). ``layout="zigzag"`` (causal only): rank r owns
    chunks r and 2*world-1-r of 2*world equal chunks (``zigzag_take``), which balances the causal work: every
    rank computes half a block per hop instead of rank 0 idling and the last rank doing all of them.
    Returns (out [B,Hq,Ls,D] in q's dtype, lse [B,Hq,Ls] fp32) for the local queries over the
    whole sequence. ``attention_fn(q, k, v, is_causal=, scale=) -> (out, lse)`` and ``merge_fn``
    default to this library's kernels. ``exchange=False`` runs the same kernels hop by hop on the local slice
    without sending anything: a timing aid that shows what the kernels cost without the transfers (its
    result is not attention over the whole sequence). ``sm_margin`` (with the default ``attention_fn``) keeps that
    many SMs out of the persistent forward kernel, so that the send/receive kernels of the hop in flight find SMs
    to run on beside it instead of waiting for it to finish."""
    if layout == "zigzag":
        if not is_causal:
            layout = "contiguous"  # without a mask every slice order is balanced and equivalent
        else:
            return _ring_prefill_zigzag(q, k, v, scale, group, attention_fn, merge_fn, exchange, sm_margin)
    elif layout != "contiguous":
        raise ValueError(f"unknown layout {layout!r}")
    if attention_fn is None:
        from . import ops
        attention_fn = functools.partial(ops.gqa_prefill, sm_margin=sm_margin)
    if merge_fn is None:
        merge_fn = merge_partial
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    B, Hq, Ls, D = q.shape
    o_acc = torch.empty((B, Hq, Ls, D), dtype=torch.float32, device=q.device)
    lse_acc = torch.full((B, Hq, Ls), float("-inf"), dtype=torch.float32, device=q.device)
    k_cur, v_cur = k.contiguous(), v.contiguous()
    send_to = dist.get_global_rank(group, (rank + 1) % world) if group is not None else (rank + 1) % world
    recv_from = dist.get_global_rank(group, (rank - 1) % world) if group is not None else (rank - 1) % world
    for step in range(world):
        src = (rank - step) % world  # owner of the slice now visiting
        reqs = []
        if step + 1 < world and exchange:
            k_next, v_next = torch.empty_like(k_cur), torch.empty_like(v_cur)
            ops_list = [dist.P2POp(dist.isend, k_cur, send_to, group), dist.P2POp(dist.isend, v_cur, send_to, group),
                        dist.P2POp(dist.irecv, k_next, recv_from, group), dist.P2POp(dist.irecv, v_next, recv_from, group)]
            reqs = dist.batch_isend_irecv(ops_list)
        if not is_causal or src <= rank:
            o_part, lse_part = attention_fn(q, k_cur, v_cur, is_causal=bool(is_causal and src == rank), scale=scale)
            merge_fn(o_acc, lse_acc, o_part, lse_part.contiguous())
        for r in reqs:
            r.wait()
        if step + 1 < world and exchange:
            k_cur, v_cur = k_next, v_next
    lse = torch.where(torch.isneginf(lse_acc), torch.full_like(lse_acc, float("inf")), lse_acc)
    return o_acc.to(q.dtype), lse


def _ring_prefill_zigzag(q, k, v, scale, group, attention_fn, merge_fn, exchange=True, sm_margin=0):
    """Causal ring prefill over zig-zag slices. Local rows are [chunk r | chunk 2W-1-r]; a visiting slice from
    rank s is [chunk s | chunk 2W-1-s]. Which parts meet:
      s == r : plain causal attention over the local slice (its two chunks are in sequence order);
      s <  r : every local query sees chunk s and nothing of chunk 2W-1-s -> all queries x first half of K/V;
      s >  r : chunk r sees nothing, chunk 2W-1-r sees both visiting chunks -> second half of queries x all K/V.
    Either way a hop is half a block of unmasked work."""
    if attention_fn is None:
        from . import ops
        attention_fn = functools.partial(ops.gqa_prefill, sm_margin=sm_margin)
    if merge_fn is None:
        merge_fn = merge_partial
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    B, Hq, Ls, D = q.shape
    assert Ls % 2 == 0, "a zig-zag slice holds two chunks of equal length"
    h = Ls // 2
    dev = q.device
    acc = [torch.empty((B, Hq, h, D), dtype=torch.float32, device=dev) for _ in range(2)]
    lse = [torch.full((B, Hq, h), float("-inf"), dtype=torch.float32, device=dev) for _ in range(2)]
    k_cur, v_cur = k.contiguous(), v.contiguous()
    send_to = dist.get_global_rank(group, (rank + 1) % world) if group is not None else (rank + 1) % world
    recv_from = dist.get_global_rank(group, (rank - 1) % world) if group is not None else (rank - 1) % world
    for step in range(world):
        src = (rank - step) % world
        reqs = []
        if step + 1 < world and exchange:
            k_next, v_next = torch.empty_like(k_cur), torch.empty_like(v_cur)
            ops_list = [dist.P2POp(dist.isend, k_cur, send_to, group), dist.P2POp(dist.isend, v_cur, send_to, group),
                        dist.P2POp(dist.irecv, k_next, recv_from, group), dist.P2POp(dist.irecv, v_next, recv_from, group)]
            reqs = dist.batch_isend_irecv(ops_list)
        if src == rank:
            o_part, l_part = attention_fn(q, k_cur, v_cur, is_causal=True, scale=scale)
            halves = (0, 1)
        elif src < rank:
            o_part, l_part = attention_fn(q, k_cur[:, :, :h], v_cur[:, :, :h], is_causal=False, scale=scale)
            halves = (0, 1)
        else:
            o_part, l_part = attention_fn(q[:, :, h:], k_cur, v_cur, is_causal=False, scale=scale)
            halves = (1,)
        for n, half in enumerate(halves):
            rows = slice(n * h, (n + 1) * h)
            merge_fn(acc[half], lse[half], o_part[:, :, rows], l_part[:, :, rows].contiguous())
        for r in reqs:
            r.wait()
        if step + 1 < world and exchange:
            k_cur, v_cur = k_next, v_next
    o_acc, lse_acc = torch.cat(acc, dim=2), torch.cat(lse, dim=2)
    lse_out = torch.where(torch.isneginf(lse_acc), torch.full_like(lse_acc, float("inf")), lse_acc)
    return o_acc.to(q.dtype), lse_out
