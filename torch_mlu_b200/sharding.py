"""Multi-GPU partitioning of the attention workloads: one process per GPU, no data-path
collective (attention is independent per batch element and per KV-head group); a single
all-gather over NCCL reassembles outputs where the caller wants them replicated.

The reference runs this operator on one device only; its collectives live in ProcessGroupCNCL
(torch_mlu/csrc/framework/distributed/process_group_cncl.cpp, ``_allgather_base`` at :1765-1818).
The equivalent used here is ``torch.distributed.all_gather_into_tensor`` on the NCCL backend
(gloo on CPU in the tests).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Sequence, Tuple

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class DenseShard:
    """Contiguous range of (batch, kv-head) units owned by one rank. Units are numbered
    b * heads_kv + hkv; a unit carries all heads_q/heads_kv query heads of its KV head, so a
    GQA group never straddles ranks."""
    unit_begin: int
    unit_end: int


def partition_units(num_units: int, world: int) -> List[DenseShard]:
    """Split ``num_units`` into ``world`` contiguous, near-equal ranges (first ranks get the
    remainder). Some ranges are empty when world > num_units."""
    base, rem = divmod(num_units, world)
    out, start = [], 0
    for r in range(world):
        n = base + (1 if r < rem else 0)
        out.append(DenseShard(start, start + n))
        start += n
    return out


def dense_shard_views(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, shard: DenseShard
                      ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Views (no copies) of q [B,Hq,L,D], k/v [B,Hkv,L,D] for one shard, flattened to a batch of
    units: q -> [units, G, L, D], k/v -> [units, 1, L, D], G = Hq/Hkv."""
    B, Hq, Lq, D = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    qf = q.reshape(B * Hkv, G, Lq, D) if q.is_contiguous() else q.contiguous().reshape(B * Hkv, G, Lq, D)
    kf = k.reshape(B * Hkv, 1, k.shape[2], D) if k.is_contiguous() else k.contiguous().reshape(B * Hkv, 1, k.shape[2], D)
    vf = v.reshape(B * Hkv, 1, v.shape[2], D) if v.is_contiguous() else v.contiguous().reshape(B * Hkv, 1, v.shape[2], D)
    s = slice(shard.unit_begin, shard.unit_end)
    return qf[s], kf[s], vf[s]


def plan_varlen(seqlens: Sequence[int], heads_kv: int, world: int) -> List[List[Tuple[int, int]]]:
    """Longest-processing-time bin packing of (sequence, kv-head) units onto ranks, cost ~ L^2
    (causal prefill work). Returns per rank a list of (sequence index, kv head)."""
    units = [(l * l, i, h) for i, l in enumerate(seqlens) for h in range(heads_kv)]
    units.sort(key=lambda u: (-u[0], u[1], u[2]))
    loads = [0] * world
    plan: List[List[Tuple[int, int]]] = [[] for _ in range(world)]
    for cost, i, h in units:
        r = min(range(world), key=lambda x: (loads[x], x))
        loads[r] += cost
        plan[r].append((i, h))
    return plan


def plan_imbalance(seqlens: Sequence[int], heads_kv: int, world: int) -> float:
    """max rank load / mean rank load for ``plan_varlen`` (1.0 = perfectly balanced)."""
    plan = plan_varlen(seqlens, heads_kv, world)
    loads = [sum(seqlens[i] ** 2 for i, _ in p) for p in plan]
    mean = sum(loads) / world
    return max(loads) / mean if mean else 1.0


def all_gather_units(local: torch.Tensor, shards: List[DenseShard], group=None) -> torch.Tensor:
    """Reassemble per-unit results ([units_r, ...] on rank r) into [sum units, ...] on every rank
    with one all_gather_into_tensor (ranks pad to the largest shard)."""
    world = dist.get_world_size(group)
    assert len(shards) == world
    max_units = max(s.unit_end - s.unit_begin for s in shards)
    tail = tuple(local.shape[1:])
    padded = local.new_zeros((max_units,) + tail)
    padded[: local.shape[0]] = local
    flat = local.new_empty((world * max_units,) + tail)  # concatenated form: accepted by nccl and gloo
    dist.all_gather_into_tensor(flat, padded, group=group)
    gathered = flat.view((world, max_units) + tail)
    parts = [gathered[r, : shards[r].unit_end - shards[r].unit_begin] for r in range(world)]
    return torch.cat(parts, 0)


def sdpa_batch_head_sharded(q, k, v, *, is_causal: bool, scale=None, group=None,
                            attention_fn: Callable = None, gather: bool = True):
    """Every rank holds the full q/k/v (or at least its own units), computes attention for its
    contiguous range of (batch, kv-head) units with ``attention_fn(q, k, v, is_causal=, scale=)``
    -> (out, lse), and (optionally) all-gathers out/lse back to [B,Hq,L,D] / [B,Hq,L]."""
    if attention_fn is None:
        from . import ops
        attention_fn = ops.gqa_prefill
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    B, Hq, Lq, D = q.shape
    Hkv = k.shape[1]
    shards = partition_units(B * Hkv, world)
    ql, kl, vl = dense_shard_views(q, k, v, shards[rank])
    if ql.shape[0] > 0:
        out_l, lse_l = attention_fn(ql, kl, vl, is_causal=is_causal, scale=scale)
        out_l = out_l.contiguous()
    else:
        out_l = q.new_empty((0, Hq // Hkv, Lq, D))
        lse_l = q.new_empty((0, Hq // Hkv, Lq), dtype=torch.float32)
    if not gather:
        return out_l, lse_l, shards
    out = all_gather_units(out_l, shards, group).reshape(B, Hq, Lq, D)
    lse = all_gather_units(lse_l.contiguous(), shards, group).reshape(B, Hq, Lq)
    return out, lse, shards
