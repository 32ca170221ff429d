"""Ring / context-parallel prefill: the host logic (slice order, causal skipping, logsumexp fold)
on CPU ranks over gloo, with the oracle standing in for the kernels."""
import os
import socket
from datetime import timedelta

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import sdpa_oracle as orc
from torch_mlu_b200 import ring


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _attn(q, k, v, *, is_causal, scale):
    return orc.attention_math(q, k, v, causal=is_causal, scale=scale)


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=60))
    g = torch.Generator().manual_seed(9)
    B, Hq, Hkv, L, D = 2, 4, 2, 24 * world, 16
    q = torch.randn(B, Hq, L, D, generator=g).bfloat16()
    k = torch.randn(B, Hkv, L, D, generator=g).bfloat16()
    v = torch.randn(B, Hkv, L, D, generator=g).bfloat16()
    sl = slice(rank * L // world, (rank + 1) * L // world)
    results = {}
    for causal in (False, True):
        out, lse = ring.ring_prefill(q[:, :, sl].float(), k[:, :, sl].float(), v[:, :, sl].float(), is_causal=causal,
                                     attention_fn=_attn, merge_fn=ring.merge_partial_reference)
        o_ref, l_ref = orc.attention_math(q, k, v, causal=causal)
        results[causal] = (float((out - o_ref[:, :, sl]).abs().max()), float((lse - l_ref[:, :, sl]).abs().max()))
    # zig-zag layout (causal): rank r owns chunks r and 2*world-1-r
    take = lambda t: ring.zigzag_take(t, rank, world)
    out, lse = ring.ring_prefill(take(q).float(), take(k).float(), take(v).float(), is_causal=True,
                                 attention_fn=_attn, merge_fn=ring.merge_partial_reference, layout="zigzag")
    o_ref, l_ref = orc.attention_math(q, k, v, causal=True)
    results["zigzag"] = (float((out - take(o_ref)).abs().max()), float((lse - take(l_ref)).abs().max()))
    torch.save(results, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_ring_prefill_matches_full_attention_world3(tmp_path):
    world = 3
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        res = torch.load(tmp_path / f"r{r}.pt")
        for causal, (eo, el) in res.items():
            assert eo < 2e-5 and el < 2e-5, (r, causal, eo, el)


def test_zigzag_rows_cover_the_sequence_once_and_balance_the_causal_work():
    world, L = 4, 64
    seen = torch.zeros(L, dtype=torch.int32)
    work = []
    for r in range(world):
        lo, hi = ring.zigzag_rows(r, world, L)
        seen[lo] += 1
        seen[hi] += 1
        rows = torch.cat([torch.arange(L)[lo], torch.arange(L)[hi]])
        work.append(int((rows + 1).sum()))  # visible keys per query under a causal mask
    assert bool((seen == 1).all())
    assert max(work) - min(work) == 0


def test_merge_reference_handles_empty_partials():
    o_acc = torch.full((1, 1, 3, 4), 7.0)
    lse_acc = torch.full((1, 1, 3), float("-inf"))
    o_part = torch.ones(1, 1, 3, 4, dtype=torch.bfloat16)
    lse_part = torch.tensor([[[0.0, float("inf"), 1.0]]])
    ring.merge_partial_reference(o_acc, lse_acc, o_part, lse_part)
    assert torch.equal(o_acc[0, 0, 0], torch.ones(4)) and torch.equal(o_acc[0, 0, 1], torch.zeros(4))
    assert lse_acc[0, 0, 1] == float("-inf") and lse_acc[0, 0, 2] == 1.0
