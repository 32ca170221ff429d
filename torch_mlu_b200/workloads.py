"""Seeded synthetic inputs for the five benchmark / parity configurations.

All tensors are N(0,1) draws from a CPU ``torch.Generator`` (so the same values exist on any
machine), cast to bf16 where the configuration says so. ``scale`` shrinks the batch / head /
length of a configuration for tests without changing how values are drawn.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

import torch


@dataclass
class DenseCase:
    name: str
    q: torch.Tensor  # [B, Hq, Lq, D]
    k: torch.Tensor  # [B, Hkv, Lk, D]
    v: torch.Tensor
    dout: Optional[torch.Tensor]
    causal: bool
    softmax_scale: float

    def forward_flops(self) -> float:
        b, hq, lq, d = self.q.shape
        lk = self.k.shape[2]
        f = 4.0 * b * hq * lq * lk * d
        return f / 2 if (self.causal and lq == lk) else f


@dataclass
class VarlenCase:
    name: str
    q: torch.Tensor  # [total, Hq, D]
    k: torch.Tensor  # [total, Hkv, D]
    v: torch.Tensor
    seqlens: List[int]
    cu_seqlens: torch.Tensor  # int32 [B+1]
    causal: bool
    softmax_scale: float

    def forward_flops(self) -> float:
        hq, d = self.q.shape[1], self.q.shape[2]
        f = sum(4.0 * hq * l * l * d for l in self.seqlens)
        return f / 2 if self.causal else f


def _randn(gen, shape, dtype):
    return torch.randn(shape, generator=gen, dtype=torch.float32).to(dtype)


def config1_cpu_reference(batch=2, heads=8, seqlen=256, head_dim=64) -> DenseCase:
    """fp32, non-causal, seed 0: the reference's own CPU-runnable case."""
    g = torch.Generator().manual_seed(0)
    q = _randn(g, (batch, heads, seqlen, head_dim), torch.float32)
    k = _randn(g, (batch, heads, seqlen, head_dim), torch.float32)
    v = _randn(g, (batch, heads, seqlen, head_dim), torch.float32)
    return DenseCase("c1_cpu_reference_fp32", q, k, v, None, False, 1.0 / math.sqrt(head_dim))


def config2_causal_prefill(batch=4, heads=32, seqlen=4096, head_dim=128, seed=1) -> DenseCase:
    """bf16 causal prefill forward, seed 1 (other seeds: further batch slices of a multi-GPU job, drawn the same way)."""
    g = torch.Generator().manual_seed(seed)
    q = _randn(g, (batch, heads, seqlen, head_dim), torch.bfloat16)
    k = _randn(g, (batch, heads, seqlen, head_dim), torch.bfloat16)
    v = _randn(g, (batch, heads, seqlen, head_dim), torch.bfloat16)
    return DenseCase("c2_causal_prefill_bf16", q, k, v, None, True, 1.0 / math.sqrt(head_dim))


def config3_causal_fwd_bwd(batch=8, heads=16, seqlen=2048, head_dim=128) -> DenseCase:
    """bf16 causal forward+backward, seed 2; q, k, v, dO drawn in that order."""
    g = torch.Generator().manual_seed(2)
    q = _randn(g, (batch, heads, seqlen, head_dim), torch.bfloat16)
    k = _randn(g, (batch, heads, seqlen, head_dim), torch.bfloat16)
    v = _randn(g, (batch, heads, seqlen, head_dim), torch.bfloat16)
    dout = _randn(g, (batch, heads, seqlen, head_dim), torch.bfloat16)
    return DenseCase("c3_causal_fwd_bwd_bf16", q, k, v, dout, True, 1.0 / math.sqrt(head_dim))


def config4_varlen_gqa(num_seqs=16, lo=512, hi=4096, heads_q=32, heads_kv=8, head_dim=128) -> VarlenCase:
    """bf16 varlen GQA causal prefill, seed 3: lengths first (uniform ints in [lo, hi]), then
    q, k, v."""
    g = torch.Generator().manual_seed(3)
    lens = torch.randint(lo, hi + 1, (num_seqs,), generator=g).tolist()
    total = sum(lens)
    q = _randn(g, (total, heads_q, head_dim), torch.bfloat16)
    k = _randn(g, (total, heads_kv, head_dim), torch.bfloat16)
    v = _randn(g, (total, heads_kv, head_dim), torch.bfloat16)
    cu = torch.zeros(num_seqs + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(lens, dtype=torch.int32).cumsum(0)
    return VarlenCase("c4_varlen_gqa_causal_bf16", q, k, v, lens, cu, True, 1.0 / math.sqrt(head_dim))


# lengths the seed-3 draw yields at the full configuration (asserted by the tests)
CONFIG4_SEQLENS = [4038, 925, 1269, 944, 597, 1532, 617, 3277, 2853, 3891, 2121, 3503, 577, 1156, 3758, 2946]


def config5_decode(batch=64, heads_q=32, heads_kv=8, seqlen_k=32768, head_dim=128, device=None) -> DenseCase:
    """bf16 split-KV decode, seed 4; drawn per batch element (q_b, k_b, v_b) so host memory
    stays bounded. With ``device`` set, each element is moved there as it is drawn."""
    g = torch.Generator().manual_seed(4)
    dev = device or "cpu"
    q = torch.empty((batch, heads_q, 1, head_dim), dtype=torch.bfloat16, device=dev)
    k = torch.empty((batch, heads_kv, seqlen_k, head_dim), dtype=torch.bfloat16, device=dev)
    v = torch.empty((batch, heads_kv, seqlen_k, head_dim), dtype=torch.bfloat16, device=dev)
    for b in range(batch):
        q[b] = _randn(g, (heads_q, 1, head_dim), torch.bfloat16).to(dev)
        k[b] = _randn(g, (heads_kv, seqlen_k, head_dim), torch.bfloat16).to(dev)
        v[b] = _randn(g, (heads_kv, seqlen_k, head_dim), torch.bfloat16).to(dev)
    return DenseCase("c5_splitkv_decode_bf16", q, k, v, None, False, 1.0 / math.sqrt(head_dim))


def decode_kv_bytes(case: DenseCase) -> int:
    """Algorithmic HBM bytes of one decode pass: K and V read once."""
    return 2 * case.k.numel() * case.k.element_size()
