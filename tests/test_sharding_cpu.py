"""Host-side logic of the multi-GPU path on CPU ranks (gloo, world_size 2): unit partitioning,
shard views, the all-gather reassembly and a rank that never joins (bounded by a short
process-group timeout instead of a hang)."""
import os
import socket
from datetime import timedelta

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import sdpa_oracle as orc
from torch_mlu_b200 import sharding, workloads


def test_partition_units_covers_everything():
    for n, w in ((128, 8), (10, 4), (3, 8), (64, 1)):
        shards = sharding.partition_units(n, w)
        assert shards[0].unit_begin == 0 and shards[-1].unit_end == n
        assert all(a.unit_end == b.unit_begin for a, b in zip(shards, shards[1:]))
        sizes = [s.unit_end - s.unit_begin for s in shards]
        assert max(sizes) - min(sizes) <= 1


def test_varlen_plan_is_balanced_for_the_benchmark_lengths():
    lens = workloads.CONFIG4_SEQLENS
    for world in (1, 2, 4, 8):
        plan = sharding.plan_varlen(lens, 8, world)
        units = sorted(u for p in plan for u in p)
        assert units == sorted((i, h) for i in range(16) for h in range(8))
        assert sharding.plan_imbalance(lens, 8, world) < 1.05


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _cpu_attention(q, k, v, *, is_causal, scale):
    out, lse = orc.attention_math(q, k, v, causal=is_causal, scale=scale)
    return out, lse


def _worker(rank, world, port, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=60))
    g = torch.Generator().manual_seed(5)
    q = torch.randn(3, 4, 40, 16, generator=g)
    k = torch.randn(3, 2, 40, 16, generator=g)
    v = torch.randn(3, 2, 40, 16, generator=g)
    out, lse, shards = sharding.sdpa_batch_head_sharded(q, k, v, is_causal=True, attention_fn=_cpu_attention)
    ref_o, ref_l = orc.attention_math(q, k, v, causal=True)
    ok = torch.allclose(out, ref_o, atol=1e-6) and torch.allclose(lse, ref_l, atol=1e-6)
    own = shards[rank].unit_end - shards[rank].unit_begin
    torch.save({"ok": bool(ok), "own": own}, os.path.join(result_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_batch_head_sharding_world2_gloo(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    res = [torch.load(tmp_path / f"r{r}.pt") for r in range(2)]
    assert all(r["ok"] for r in res)
    assert sum(r["own"] for r in res) == 3 * 2


def _lonely_worker(rank, world, port, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=3))
    if rank == 1:
        # this rank leaves between steps, with nothing in flight
        dist.destroy_process_group()
        return
    x = torch.ones(4)
    try:
        dist.all_reduce(x)
        outcome = "completed"
    except Exception as e:  # the short timeout turns the missing peer into an error, not a hang
        outcome = "error:" + type(e).__name__
    torch.save({"outcome": outcome}, os.path.join(result_dir, "lonely.pt"))


def test_missing_rank_surfaces_as_an_error_not_a_hang(tmp_path):
    port = _free_port()
    mp.spawn(_lonely_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    res = torch.load(tmp_path / "lonely.pt")
    assert res["outcome"].startswith("error:")
