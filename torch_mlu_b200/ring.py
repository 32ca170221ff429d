"""Ring / context-parallel prefill for sequences too long for one GPU's share of the work.

Every rank owns a contiguous slice of the sequence: its queries stay put, the key/value slices
travel around the ring (``batch_isend_irecv`` over NCCL: each hop lands in this GPU's own memory
before any kernel reads it). At every hop the local forward kernel produces a partial
(out, logsumexp) for (local queries x visiting keys) and ``merge_partial`` folds it into an fp32
accumulator by the logsumexp rule. Causal masking falls out of the slice order: a visiting slice
from an earlier rank is fully visible, the rank's own slice is the usual lower triangle, slices
from later ranks are skipped (but still forwarded).

``exchange="peer"`` moves the slices another way: every rank keeps its visiting slice in one of two buffers that
its right-hand neighbour has mapped through CUDA IPC, and a hop is a plain device-to-device copy that the neighbour
pulls with the copy engines over NVLink (716 GB/s measured, against 135-147 GB/s per direction for the send/receive
pair, and no SM taken from the attention kernel); one one-word all-reduce per hop orders the ranks. The copy lands in
this GPU's own memory before any kernel reads it, as before.

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


class _PeerRing:
    """Two (K, V) buffer pairs per rank plus the left-hand neighbour's two pairs, mapped through CUDA IPC.

    Hop s: this rank's attention reads pair s % 2; meanwhile the pair (s + 1) % 2 receives the left neighbour's pair
    s % 2 by a copy on `stream`. Before that copy every rank must (a) hold its slice of step s in pair s % 2 and
    (b) have nobody reading pair (s + 1) % 2 any more - its own attention of step s - 1, and the right neighbour's
    copy of hop s - 1. (a) and the neighbour's part of (b) are what the all-reduce in front of the copy waits for:
    each rank enters it only behind its own copy of hop s - 1."""

    def __init__(self, k: torch.Tensor, v: torch.Tensor, group):
        dev = k.device
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        self.shape_k, self.shape_v, self.dtype = tuple(k.shape), tuple(v.shape), k.dtype
        self.k = [torch.empty(k.shape, dtype=k.dtype, device=dev) for _ in range(2)]
        self.v = [torch.empty(v.shape, dtype=v.dtype, device=dev) for _ in range(2)]
        self.stamp = torch.full((4,), float(rank), dtype=torch.float32, device=dev)
        mine = []
        for t in (self.k[0], self.v[0], self.k[1], self.v[1], self.stamp):
            mine.append((t.untyped_storage()._share_cuda_(), t.storage_offset(), tuple(t.shape), t.dtype))
        everyone = [None] * world
        dist.all_gather_object(everyone, mine, group=group)
        left = (rank - 1) % world
        self._peer_storages = []
        peer = []
        for handle, offset, shape, dtype in everyone[left]:
            st = torch.UntypedStorage._new_shared_cuda(*handle)
            self._peer_storages.append(st)
            peer.append(torch.empty(0, dtype=dtype, device=st.device).set_(st, offset, shape))
        self.peer_k, self.peer_v = [peer[0], peer[2]], [peer[1], peer[3]]
        # the mapping must really be the left neighbour's memory (it is not when the processes number the GPUs
        # differently, e.g. each with its own CUDA_VISIBLE_DEVICES)
        seen = float(peer[4].to(dev)[0].item())
        if seen != float(left):
            raise RuntimeError(f"CUDA IPC mapping of rank {left}'s buffers shows rank {seen:.0f}'s data")
        self.stream = torch.cuda.Stream(dev)
        self.word = torch.zeros(1, dtype=torch.float32, device=dev)
        dist.barrier(group=group)

    def release(self):
        self.peer_k = self.peer_v = None
        self._peer_storages = None


_peer_rings: dict = {}


def _peer_ring(k: torch.Tensor, v: torch.Tensor, group) -> _PeerRing:
    key = (k.device.index, tuple(k.shape), tuple(v.shape), k.dtype, id(group))
    ring_ = _peer_rings.get(key)
    if ring_ is None:
        ring_ = _peer_rings[key] = _PeerRing(k, v, group)
    return ring_


def release_peer_buffers(group=None) -> None:
    """Unmaps the neighbours' buffers (call on every rank before the process group goes away)."""
    for ring_ in _peer_rings.values():
        ring_.release()
    _peer_rings.clear()
    if dist.is_initialized():
        dist.barrier(group=group)


class _Exchange:
    """The K/V slices of the hop loop, by one of the two transports. `current()` is the pair the step's attention reads;
    `start_next(step)` starts moving the next pair in, `finish_next()` makes the compute stream wait for it."""

    def __init__(self, k, v, group, mode):
        self.group, self.mode = group, mode
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.k_cur, self.v_cur = k.contiguous(), v.contiguous()
        self.reqs = []
        if mode == "peer":
            self.ring = _peer_ring(self.k_cur, self.v_cur, group)
            # the right neighbour may still be copying out of pair 0 for the previous call's first hop: every rank
            # comes here behind its own copies of that call, so this all-reduce puts the new slice behind them all
            dist.all_reduce(self.ring.word, group=group)
            self.ring.k[0].copy_(self.k_cur)
            self.ring.v[0].copy_(self.v_cur)
            self.k_cur, self.v_cur = self.ring.k[0], self.ring.v[0]
            self.step_done = torch.cuda.Event()
            self.step_done.record()
        elif mode:
            to_global = (lambda r: dist.get_global_rank(group, r)) if group is not None else (lambda r: r)
            self.send_to, self.recv_from = to_global((self.rank + 1) % self.world), to_global((self.rank - 1) % self.world)

    def current(self):
        return self.k_cur, self.v_cur

    def start_next(self, step):
        if step + 1 >= self.world or not self.mode:
            return
        if self.mode == "peer":
            r, cur, nxt = self.ring, step % 2, (step + 1) % 2
            with torch.cuda.stream(r.stream):
                r.stream.wait_event(self.step_done)  # pair `cur` is written, the attention that read pair `nxt` is done
                dist.all_reduce(r.word, group=self.group)
                r.k[nxt].copy_(r.peer_k[cur], non_blocking=True)
                r.v[nxt].copy_(r.peer_v[cur], non_blocking=True)
                self.pulled = torch.cuda.Event()
                self.pulled.record()
            self.k_next, self.v_next = r.k[nxt], r.v[nxt]
        else:
            self.k_next, self.v_next = torch.empty_like(self.k_cur), torch.empty_like(self.v_cur)
            g = self.group
            self.reqs = dist.batch_isend_irecv([dist.P2POp(dist.isend, self.k_cur, self.send_to, g),
                                                dist.P2POp(dist.isend, self.v_cur, self.send_to, g),
                                                dist.P2POp(dist.irecv, self.k_next, self.recv_from, g),
                                                dist.P2POp(dist.irecv, self.v_next, self.recv_from, g)])

    def finish_next(self, step):
        if step + 1 >= self.world or not self.mode:
            return
        if self.mode == "peer":
            self.step_done = torch.cuda.Event()
            self.step_done.record()  # this step's attention (and merge) are behind this point of the compute stream
            torch.cuda.current_stream().wait_event(self.pulled)
        else:
            for r in self.reqs:
                r.wait()
            self.reqs = []
        self.k_cur, self.v_cur = self.k_next, self.v_next


def ring_prefill(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, is_causal: bool, scale: Optional[float] = None,
                 group=None, attention_fn: Optional[Callable] = None, merge_fn: Optional[Callable] = None,
                 layout: str = "contiguous", exchange=True, sm_margin: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
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
    to run on beside it instead of waiting for it to finish. ``exchange="peer"`` pulls the slices with copy-engine
    copies from the neighbour's IPC-mapped buffers instead (see the module text); the one-word all-reduce per hop still
    is a kernel, so at least four SMs are left free then. Call ``release_peer_buffers()`` before the process group
    is destroyed."""
    if exchange == "peer":
        sm_margin = max(int(sm_margin), 4)
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
    ex = _Exchange(k, v, group, exchange)
    for step in range(world):
        src = (rank - step) % world  # owner of the slice now visiting
        k_cur, v_cur = ex.current()
        ex.start_next(step)
        if not is_causal or src <= rank:
            o_part, lse_part = attention_fn(q, k_cur, v_cur, is_causal=bool(is_causal and src == rank), scale=scale)
            merge_fn(o_acc, lse_acc, o_part, lse_part.contiguous())
        ex.finish_next(step)
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
    ex = _Exchange(k, v, group, exchange)
    for step in range(world):
        src = (rank - step) % world
        k_cur, v_cur = ex.current()
        ex.start_next(step)
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
        ex.finish_next(step)
    o_acc, lse_acc = torch.cat(acc, dim=2), torch.cat(lse, dim=2)
    lse_out = torch.where(torch.isneginf(lse_acc), torch.full_like(lse_acc, float("inf")), lse_acc)
    return o_acc.to(q.dtype), lse_out
