"""Host-resident inputs and outputs: a double-buffered copy / compute / copy pipeline around the
prefill operator.

A caller whose q, k, v live in (pinned) host memory and whose results go back to the host pays PCIe
for every call; done on one stream, the three phases add up. ``HostPipeline`` keeps two sets of device
buffers and three streams, so that call i+1's host-to-device copies, call i's kernel and call i-1's
device-to-host copies overlap. Every call still moves all of its inputs in and all of its results
out; only the waiting is shared. The reference has no counterpart (its tensors live on the device,
copies are the caller's business: torch_mlu/csrc/framework/core/memory_allocator.cpp is its pinned
host allocator); this is the serving-side plumbing bench.py's end-to-end figure is measured through.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from . import ops


class HostPipeline:
    """Dense causal/non-causal prefill for fixed shapes, host tensors in and out.

    ``submit(q, k, v, out, lse)`` enqueues one call: q [B,Hq,Lq,D], k/v [B,Hkv,Lk,D] pinned host tensors
    (bf16 or fp16), ``out`` a pinned host tensor [B,Lq,Hq,D] (the memory order the operator produces),
    ``lse`` pinned fp32 [B,Hq,Lq]. Results are valid after ``wait()`` (or after the event ``submit``
    returns has completed). Host buffers must not be reused before then.
    """

    def __init__(self, device: torch.device, *, is_causal: bool, scale: Optional[float] = None, depth: int = 2):
        if depth < 2:
            raise ValueError("depth must be at least 2 (one buffer set being filled, one being used)")
        self.device = device
        self.is_causal = is_causal
        self.scale = scale
        self.depth = depth
        self.h2d = torch.cuda.Stream(device)
        self.compute = torch.cuda.Stream(device)
        self.d2h = torch.cuda.Stream(device)
        self._in: List[Optional[Tuple[torch.Tensor, ...]]] = [None] * depth
        self._out: List[Optional[Tuple[torch.Tensor, torch.Tensor]]] = [None] * depth
        self._in_free: List[Optional[torch.cuda.Event]] = [None] * depth   # kernel that read the inputs is done
        self._out_done: List[Optional[torch.cuda.Event]] = [None] * depth  # results of that slot are on the host
        self._n = 0

    def submit(self, q, k, v, out, lse) -> torch.cuda.Event:
        for t in (q, k, v, out, lse):
            if not t.is_pinned():
                raise ValueError("HostPipeline needs pinned host tensors (pageable memory makes the copies synchronous)")
        s = self._n % self.depth
        self._n += 1
        with torch.cuda.stream(self.h2d):
            if self._in_free[s] is not None:
                self.h2d.wait_event(self._in_free[s])
            if self._in[s] is None or self._in[s][0].shape != q.shape or self._in[s][1].shape != k.shape \
                    or self._in[s][0].dtype != q.dtype:
                self._in[s] = tuple(torch.empty(t.shape, dtype=t.dtype, device=self.device) for t in (q, k, v))
            qd, kd, vd = self._in[s]
            qd.copy_(q, non_blocking=True)
            kd.copy_(k, non_blocking=True)
            vd.copy_(v, non_blocking=True)
            in_ready = torch.cuda.Event()
            in_ready.record(self.h2d)
        with torch.cuda.stream(self.compute):
            self.compute.wait_event(in_ready)
            if self._out_done[s] is not None:
                self.compute.wait_event(self._out_done[s])  # the slot's previous results have left the device
            o, l = ops.gqa_prefill(qd, kd, vd, is_causal=self.is_causal, scale=self.scale)
            self._out[s] = (o, l)  # keeps the device tensors alive until the slot is reused
            done = torch.cuda.Event()
            done.record(self.compute)
            self._in_free[s] = done
        with torch.cuda.stream(self.d2h):
            self.d2h.wait_event(done)
            out.copy_(o.transpose(1, 2), non_blocking=True)
            lse.copy_(l, non_blocking=True)
            out_done = torch.cuda.Event()
            out_done.record(self.d2h)
            self._out_done[s] = out_done
        return out_done

    def wait(self) -> None:
        """Block the host until everything submitted so far is back in host memory."""
        for e in self._out_done:
            if e is not None:
                e.synchronize()

    def join(self, stream: Optional[torch.cuda.Stream] = None) -> None:
        """Make ``stream`` (default: the current one) wait for everything submitted so far."""
        stream = stream or torch.cuda.current_stream(self.device)
        for e in self._out_done:
            if e is not None:
                stream.wait_event(e)
