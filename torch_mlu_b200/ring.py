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
pair, and no SM taken from the attention kernel). Neighbours order their hops through two counters each, written and
waited for by the streams themselves (cuStreamWriteValue32 / cuStreamWaitValue32: "my slice for hop n is in place",
"I have copied hop n out of your buffer"), or, where those are not available, by a one-word all-reduce per hop. The copy lands in
this GPU's own memory before any kernel reads it, as before.

The reference has no such path (its attention is single-device; P2P lives in
ProcessGroupCNCL::send/recv, process_group_cncl.cpp:2526-2552).
"""
from __future__ import annotations

import ctypes
import functools
import time
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
    """Two (K, V) buffer pairs per rank, the left-hand neighbour's two pairs and both neighbours' counters, mapped
    through CUDA IPC.

    Hop n (counted over all calls): this rank's attention reads its source pair; meanwhile the other pair receives the
    left neighbour's source pair by copies on `stream`. Before those copies (a) the left neighbour must hold its slice
    for this hop in its source pair and (b) nobody may be reading the destination pair any more - this rank's own
    attention of the step before (an event), and the right neighbour's copies of hop n - 1. Each rank therefore keeps
    two counters that its neighbours write: flags[0] <- n from the left ("my slice for hop n is in place"), flags[1] <- n
    from the right ("I have copied hop n out of your buffer"); its stream waits for flags[0] >= n and flags[1] >= n - 1
    before it copies, and a call waits for flags[1] >= (hops so far) before it overwrites a pair with its own slice.
    Where the streams cannot do that themselves (`memops` false) a one-word all-reduce in front of every hop's copies
    stands for both conditions: each rank enters it only behind its own copies of the hop before."""

    def __init__(self, k: torch.Tensor, v: torch.Tensor, group):
        dev = k.device
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        self.shape_k, self.shape_v, self.dtype = tuple(k.shape), tuple(v.shape), k.dtype
        self.k = [torch.empty(k.shape, dtype=k.dtype, device=dev) for _ in range(2)]
        self.v = [torch.empty(v.shape, dtype=v.dtype, device=dev) for _ in range(2)]
        self.stamp = torch.full((4,), float(rank), dtype=torch.float32, device=dev)
        # [0] written by the left neighbour: the number of the last hop whose source pair over there is valid;
        # [1] written by the right neighbour: the number of the last hop it has finished copying out of this rank;
        # [2], [3]: the set-up's own check that such writes arrive
        self.flags = torch.zeros(4, dtype=torch.int32, device=dev)
        self.hops = 0  # hops made so far, over all calls (the same number on every rank)
        self.pair = 0  # the pair the next call puts its own slice in
        # Every step below that can fail is followed by an agreement among the ranks, so that they all go on or all
        # raise: a rank that gave up alone would leave the others waiting in the next collective.
        try:
            mine, error = [], None
            for t in (self.k[0], self.v[0], self.k[1], self.v[1], self.stamp, self.flags):
                mine.append((t.untyped_storage()._share_cuda_(), t.storage_offset(), tuple(t.shape), t.dtype))
        except Exception as e:  # noqa: BLE001 - reported below, on every rank
            mine, error = None, f"{type(e).__name__}: {e}"
        everyone = [None] * world
        dist.all_gather_object(everyone, mine, group=group)
        left = (rank - 1) % world
        self._peer_storages = []
        if error is None and all(m is not None for m in everyone):
            try:
                peer = []
                for handle, offset, shape, dtype in everyone[left]:
                    st = torch.UntypedStorage._new_shared_cuda(*handle)
                    self._peer_storages.append(st)
                    peer.append(torch.empty(0, dtype=dtype, device=st.device).set_(st, offset, shape))
                self.peer_k, self.peer_v = [peer[0], peer[2]], [peer[1], peer[3]]
                self.left_flags = peer[5]
                handle, offset, shape, dtype = everyone[(rank + 1) % world][5]
                st = torch.UntypedStorage._new_shared_cuda(*handle)
                self._peer_storages.append(st)
                self.right_flags = torch.empty(0, dtype=dtype, device=st.device).set_(st, offset, shape)
                # the mapping must really be the left neighbour's memory (it is not when the processes number the
                # GPUs differently, e.g. each with its own CUDA_VISIBLE_DEVICES)
                seen = float(peer[4].to(dev)[0].item())
                if seen != float(left):
                    error = f"CUDA IPC mapping of rank {left}'s buffers shows rank {seen:.0f}'s data"
            except Exception as e:  # noqa: BLE001
                error = f"{type(e).__name__}: {e}"
        elif error is None:
            error = "another rank could not export its buffers"
        failed = torch.tensor([0.0 if error is None else 1.0], device=dev)
        dist.all_reduce(failed, group=group)
        if failed.item() != 0.0:
            self.release()
            raise RuntimeError(f"peer-copy ring exchange unavailable on {int(failed.item())} rank(s)"
                               + (f"; here: {error}" if error else ""))
        self.stream = torch.cuda.Stream(dev)
        self.word = torch.zeros(1, dtype=torch.float32, device=dev)
        dist.barrier(group=group)
        # Ordering between neighbours without any kernel: 32-bit writes and waits that the stream itself performs
        # (cuStreamWriteValue32 / cuStreamWaitValue32). Tried once here, a write into the right neighbour's flags and a
        # wait for the left neighbour's; if any rank cannot, every rank orders its hops with a one-word all-reduce.
        self.memops = self._try_memops(dev, group)
        self.broken = False
        self._rescue = torch.cuda.Stream(dev)
        self._all_ones = torch.full((2,), 0x7fffffff, dtype=torch.int32, device=dev)

    _CU_WAIT_GEQ = 0x0

    def _try_memops(self, dev, group) -> bool:
        ok = True
        try:
            lib = ctypes.CDLL("libcuda.so.1")
            self._cu_wait = getattr(lib, "cuStreamWaitValue32_v2", None) or lib.cuStreamWaitValue32
            self._cu_write = getattr(lib, "cuStreamWriteValue32_v2", None) or lib.cuStreamWriteValue32
            for fn in (self._cu_wait, self._cu_write):
                fn.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_uint]
                fn.restype = ctypes.c_int
            # Copies are issued on THIS GPU's stream (torch issues a copy between devices on the source's, which here
            # would be this process's context on the neighbour's GPU: it then waits for a time slice between the
            # neighbour's own kernels, ~0.5 ms per hop).
            self._memcpy = ctypes.CDLL("libcudart.so.12").cudaMemcpyAsync
            self._memcpy.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]
            self._memcpy.restype = ctypes.c_int
            self.stage = torch.zeros(2, dtype=torch.int32, device=dev)  # the words that travel to the neighbours
            with torch.cuda.device(dev), torch.cuda.stream(self.stream):
                self.post(self.stream, self.right_flags, 2, 7, 0)     # lands in the right neighbour's flags[2]
                self.write_flag(self.stream, self.flags, 3, 9)
                self.wait_flag(self.stream, self.flags, 3, 9)         # already true: this probe cannot wait for ever
            self.stream.synchronize()
        except Exception as e:  # noqa: BLE001 - any failure means: use the all-reduce
            ok, self.memops_note = False, f"{type(e).__name__}: {e}"
        dist.barrier(group=group)  # every rank's write into its neighbour has been performed
        if ok:
            got = (int(self.flags[2].item()), int(self.flags[3].item()))
            ok = got == (7, 9)
            self.memops_note = "" if ok else f"flags read back {got}, expected (7, 9)"
        agreed = torch.tensor([1.0 if ok else 0.0], device=dev)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=group)
        return bool(agreed.item() == 1.0)

    def post(self, stream, peer_flags: torch.Tensor, index: int, value: int, word: int) -> None:
        """`value` into a neighbour's flag, in stream order: the stream writes it into a word of this GPU's memory
        (stream memory operations do not take a peer's address) and a four-byte peer copy carries it over. Call with
        `stream` current."""
        self.write_flag(stream, self.stage, word, value)
        self.copy(stream, peer_flags[index:index + 1], self.stage[word:word + 1])

    def copy(self, stream, dst: torch.Tensor, src: torch.Tensor) -> None:
        """dst <- src (contiguous, same size; either may be a neighbour's mapped memory) by cudaMemcpyAsync on `stream`."""
        err = self._memcpy(dst.data_ptr(), src.data_ptr(), dst.numel() * dst.element_size(), 4, stream.cuda_stream)
        if err != 0:
            raise RuntimeError(f"cudaMemcpyAsync failed with cudaError {err}")

    def finish(self, timeout_s: float) -> None:
        """The stream waits of this transport have no time limit of their own, so every call ends with one on the host:
        if the work queued so far is not done after `timeout_s`, this rank's counters are set to their largest value
        (every wait of this rank then passes, the streams drain, the results are void) and the call raises. A
        neighbour that was waiting for this rank runs into its own limit the same way."""
        done = torch.cuda.Event()
        done.record()
        deadline = time.monotonic() + timeout_s
        while not done.query():
            if time.monotonic() > deadline:
                self.broken = True
                with torch.cuda.stream(self._rescue):
                    self.copy(self._rescue, self.flags[0:2], self._all_ones)
                self._rescue.synchronize()
                done.synchronize()
                raise RuntimeError(f"peer-copy ring exchange: a hop did not complete within {timeout_s:.0f} s; "
                                   "this rank's waits were released and its result is void")
            time.sleep(0.0002)

    def write_flag(self, stream, flags: torch.Tensor, index: int, value: int) -> None:
        err = self._cu_write(ctypes.c_void_p(stream.cuda_stream), flags.data_ptr() + 4 * index, value, 0)
        if err != 0:
            raise RuntimeError(f"cuStreamWriteValue32 failed with CUresult {err}")

    def wait_flag(self, stream, flags: torch.Tensor, index: int, value: int) -> None:
        err = self._cu_wait(ctypes.c_void_p(stream.cuda_stream), flags.data_ptr() + 4 * index, value, self._CU_WAIT_GEQ)
        if err != 0:
            raise RuntimeError(f"cuStreamWaitValue32 failed with CUresult {err}")

    def release(self):
        self.peer_k = self.peer_v = self.left_flags = self.right_flags = None
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


def peer_call_plan(world: int, hops_before: int, first_pair: int) -> dict:
    """The counter protocol of one ring call with the peer transport, as data (what `_Exchange` executes and what
    `tests/test_ring_cpu.py` replays on a model of the streams). Hops are numbered from 1 over all calls.

    `start`: before the call writes its own slice into pair `first_pair`, the compute stream waits until the right
    neighbour has copied hop `wait_free` out (None for the first call). `hops[s]` for step s < world - 1, on the
    copy stream behind the event "pair `src` is written and the attention that read pair `dst` is done":
    `announce_now` (write hop number to the right neighbour's counter 0 - a call's first hop only), wait counter 0
    >= `hop`, wait counter 1 >= `hop - 1` (`wait_free`, None for hop 1), copy the left neighbour's pair `src` into
    pair `dst`, write `hop` to the left neighbour's counter 1, and `announce_next` (hop + 1 to the right neighbour's
    counter 0: pair `dst` is the next hop's source; None on a call's last hop). `next_first_pair` is where the next call
    starts."""
    hops = []
    for step in range(world - 1):
        hop = hops_before + step + 1
        hops.append({"hop": hop, "src": (first_pair + step) % 2, "dst": (first_pair + step + 1) % 2,
                     "announce_now": step == 0, "wait_free": hop - 1 if hop > 1 else None,
                     "announce_next": hop + 1 if step + 2 < world else None})
    return {"start": {"wait_free": hops_before if hops_before > 0 else None, "pair": first_pair}, "hops": hops,
            "next_first_pair": (first_pair + world) % 2}


class _Exchange:
    """The K/V slices of the hop loop, by one of the two transports. `current()` is the pair the step's attention reads;
    `start_next(step)` starts moving the next pair in, `finish_next()` makes the compute stream wait for it."""

    def __init__(self, k, v, group, mode):
        self.group, self.mode = group, mode
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.k_cur, self.v_cur = k.contiguous(), v.contiguous()
        self.reqs = []
        if mode == "peer":
            r = self.ring = _peer_ring(self.k_cur, self.v_cur, group)
            if r.broken:
                raise RuntimeError("peer-copy ring exchange: an earlier call ran into its time limit; "
                                   "call release_peer_buffers() on every rank before using it again")
            # The pair that takes this call's own slice is the one the right neighbour copied out of in the previous
            # call's last hop: the new slice goes in behind that copy.
            if r.memops:
                self.plan = peer_call_plan(self.world, r.hops, r.pair)
                self.first = self.plan["start"]["pair"]
                r.pair = self.plan["next_first_pair"]
                if self.plan["start"]["wait_free"] is not None:
                    r.wait_flag(torch.cuda.current_stream(), r.flags, 1, self.plan["start"]["wait_free"])
            else:
                self.first = 0
                # (every rank comes here behind its own copies of the previous call)
                dist.all_reduce(r.word, group=group)
            r.k[self.first].copy_(self.k_cur)
            r.v[self.first].copy_(self.v_cur)
            self.k_cur, self.v_cur = r.k[self.first], r.v[self.first]
            self.step_done = torch.cuda.Event()
            self.step_done.record()
        elif mode:
            to_global = (lambda r: dist.get_global_rank(group, r)) if group is not None else (lambda r: r)
            self.send_to, self.recv_from = to_global((self.rank + 1) % self.world), to_global((self.rank - 1) % self.world)

    def current(self):
        return self.k_cur, self.v_cur

    def finish(self, timeout_s: float) -> None:
        if self.mode == "peer" and self.ring.memops:
            self.ring.finish(timeout_s)

    def start_next(self, step):
        if step + 1 >= self.world or not self.mode:
            return
        if self.mode == "peer":
            r, cur, nxt = self.ring, (self.first + step) % 2, (self.first + step + 1) % 2
            with torch.cuda.stream(r.stream):
                r.stream.wait_event(self.step_done)  # pair `cur` is written, the attention that read pair `nxt` is done
                if r.memops:
                    h = self.plan["hops"][step]
                    hop = h["hop"]
                    assert (h["src"], h["dst"]) == (cur, nxt) and hop == r.hops + 1
                    # to the right: my source pair of this hop is valid. Said here only for a call's first hop; for the
                    # later ones it was said as soon as the pair was filled (below), a whole step earlier, so that
                    # the neighbour's wait finds it there: a stream wait that has to wait costs ~0.35 ms.
                    if h["announce_now"]:
                        r.post(r.stream, r.right_flags, 0, hop, 0)
                    r.wait_flag(r.stream, r.flags, 0, hop)             # the left neighbour's is
                    if h["wait_free"] is not None:
                        r.wait_flag(r.stream, r.flags, 1, h["wait_free"])  # the right neighbour has left pair `nxt` alone
                else:
                    dist.all_reduce(r.word, group=self.group)
                if r.memops:
                    r.copy(r.stream, r.k[nxt], r.peer_k[cur])
                    r.copy(r.stream, r.v[nxt], r.peer_v[cur])
                else:
                    r.k[nxt].copy_(r.peer_k[cur], non_blocking=True)
                    r.v[nxt].copy_(r.peer_v[cur], non_blocking=True)
                if r.memops:
                    r.post(r.stream, r.left_flags, 1, hop, 1)          # to the left: I am done with your pair
                    if h["announce_next"] is not None:
                        r.post(r.stream, r.right_flags, 0, h["announce_next"], 0)  # pair `nxt` is the next hop's source
                    r.hops = hop
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
                 layout: str = "contiguous", exchange=True, sm_margin: Optional[int] = None,
                 peer_timeout_s: float = 30.0) -> Tuple[torch.Tensor, torch.Tensor]:
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
    to run on beside it instead of waiting for it to finish; left at None it is 16 for the send/receive ring on more
    than two ranks (measured best on four and eight GPUs; on two the hop's kernels are long enough to hide the
    exchange anyway) and 0 otherwise. ``exchange="peer"`` pulls the slices with copy-engine
    copies from the neighbour's IPC-mapped buffers instead (see the module text); where the hops have to be ordered by a
    one-word all-reduce (no stream memory operations), that still is a kernel and at least four SMs are left free. Call ``release_peer_buffers()`` before the process group
    is destroyed. Such a call returns only when its work on the GPU is done, or raises after ``peer_timeout_s``
    (the stream waits it uses have no time limit of their own; see ``_PeerRing.finish``)."""
    if sm_margin is None:
        sm_margin = 16 if (exchange is True and dist.get_world_size(group) > 2) else 0
    if exchange == "peer" and not _peer_ring(k.contiguous(), v.contiguous(), group).memops:
        sm_margin = max(int(sm_margin), 4)
    if layout == "zigzag":
        if not is_causal:
            layout = "contiguous"  # without a mask every slice order is balanced and equivalent
        else:
            return _ring_prefill_zigzag(q, k, v, scale, group, attention_fn, merge_fn, exchange, sm_margin, peer_timeout_s)
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
    out = o_acc.to(q.dtype)
    ex.finish(peer_timeout_s)
    return out, lse


def _ring_prefill_zigzag(q, k, v, scale, group, attention_fn, merge_fn, exchange=True, sm_margin=0, peer_timeout_s=30.0):
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
    out = o_acc.to(q.dtype)
    ex.finish(peer_timeout_s)
    return out, lse_out
