"""Ring / context-parallel prefill: the host logic (slice order, causal skipping, logsumexp fold)
on CPU ranks over gloo, with the oracle standing in for the kernels."""
import os
import socket
from datetime import timedelta

import pytest
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


# ---------------------------------------------------------------------------------------------------------------
# The peer transport's counter protocol (ring.peer_call_plan), replayed on a model of the streams: every rank has a
# compute stream and a copy stream that run their operations in order; a scheduler picks any operation that can run,
# at random. Copies, reads and writes take time (begin / end), so overlaps show. Checked: nothing is read while it
# is written or written while it is read, every step's attention sees the slice it should, and nobody waits for ever.
# ---------------------------------------------------------------------------------------------------------------
def _ring_streams(world, calls):
    from torch_mlu_b200 import ring
    streams = {}
    event_ids = iter(range(10 ** 9))
    state = {r: {"hops": 0, "pair": 0} for r in range(world)}
    for r in range(world):
        compute, copy = [], []
        left, right = (r - 1) % world, (r + 1) % world
        for c in range(calls):
            plan = ring.peer_call_plan(world, state[r]["hops"], state[r]["pair"])
            first = plan["start"]["pair"]
            state[r]["pair"] = plan["next_first_pair"]
            if plan["start"]["wait_free"] is not None:
                compute.append(("wait_flag", 1, plan["start"]["wait_free"]))
            compute += [("write_begin", first), ("write_end", first, (c, r))]
            step_done = next(event_ids)
            compute.append(("record", step_done))
            for step in range(world):
                cur = (first + step) % 2
                pulled = None
                if step + 1 < world:
                    h = plan["hops"][step]
                    assert h["src"] == cur
                    pulled = next(event_ids)
                    copy.append(("wait_event", step_done))
                    if h["announce_now"]:
                        copy.append(("post", right, 0, h["hop"]))
                    copy.append(("wait_flag", 0, h["hop"]))
                    if h["wait_free"] is not None:
                        copy.append(("wait_flag", 1, h["wait_free"]))
                    copy += [("copy_begin", left, h["src"], h["dst"]), ("copy_end", left, h["src"], h["dst"]),
                             ("post", left, 1, h["hop"])]
                    if h["announce_next"] is not None:
                        copy.append(("post", right, 0, h["announce_next"]))
                    copy.append(("record", pulled))
                    state[r]["hops"] = h["hop"]
                compute += [("read_begin", cur, (c, (r - step) % world)), ("read_end", cur)]
                if pulled is not None:
                    step_done = next(event_ids)
                    compute += [("record", step_done), ("wait_event", pulled)]
        streams[(r, "compute")] = compute
        streams[(r, "copy")] = copy
    return streams


def _replay(world, calls, seed):
    import random
    rng = random.Random(seed)
    streams = _ring_streams(world, calls)
    pos = {k: 0 for k in streams}
    flags = {r: [0, 0] for r in range(world)}
    events = set()
    pairs = {r: [{"label": None, "readers": 0, "writing": False, "incoming": None} for _ in range(2)] for r in range(world)}

    def can_run(key, op):
        r = key[0]
        if op[0] == "wait_flag":
            return flags[r][op[1]] >= op[2]
        if op[0] == "wait_event":
            return op[1] in events
        return True

    def run(key, op):
        r = key[0]
        kind = op[0]
        if kind == "post":
            flags[op[1]][op[2]] = max(flags[op[1]][op[2]], op[3])
        elif kind == "record":
            events.add(op[1])
        elif kind == "write_begin":
            p = pairs[r][op[1]]
            assert p["readers"] == 0 and not p["writing"], f"rank {r} overwrites pair {op[1]} in use"
            p["writing"] = True
        elif kind == "write_end":
            p = pairs[r][op[1]]
            p["writing"], p["label"] = False, op[2]
        elif kind == "copy_begin":
            src, dst = pairs[op[1]][op[2]], pairs[r][op[3]]
            assert not src["writing"], f"rank {r} copies rank {op[1]}'s pair {op[2]} while it is written"
            assert dst["readers"] == 0 and not dst["writing"], f"rank {r} copies into its pair {op[3]} in use"
            src["readers"] += 1
            dst["writing"], dst["incoming"] = True, src["label"]
        elif kind == "copy_end":
            src, dst = pairs[op[1]][op[2]], pairs[r][op[3]]
            src["readers"] -= 1
            dst["writing"], dst["label"] = False, dst["incoming"]
        elif kind == "read_begin":
            p = pairs[r][op[1]]
            assert not p["writing"], f"rank {r} reads pair {op[1]} while it is written"
            assert p["label"] == op[2], f"rank {r} reads slice {p['label']}, expected {op[2]}"
            p["readers"] += 1
        elif kind == "read_end":
            pairs[r][op[1]]["readers"] -= 1

    while True:
        ready = [k for k in streams if pos[k] < len(streams[k]) and can_run(k, streams[k][pos[k]])]
        if not ready:
            assert all(pos[k] == len(streams[k]) for k in streams), \
                f"deadlock: {[(k, streams[k][pos[k]]) for k in streams if pos[k] < len(streams[k])]}"
            return
        k = rng.choice(ready)
        run(k, streams[k][pos[k]])
        pos[k] += 1


@pytest.mark.parametrize("world", [2, 3, 4, 5, 8])
def test_peer_ring_counters_keep_copies_reads_and_writes_apart(world):
    for seed in range(150):
        _replay(world, calls=3, seed=seed)


def test_the_model_notices_a_missing_wait(monkeypatch):
    """The same replay with the "right neighbour has copied out" wait taken away must trip a check (or the model
    proves nothing)."""
    from torch_mlu_b200 import ring
    real = ring.peer_call_plan

    def careless(world, hops_before, first_pair):
        plan = real(world, hops_before, first_pair)
        plan["start"]["wait_free"] = None
        for h in plan["hops"]:
            h["wait_free"] = None
        return plan

    monkeypatch.setattr(ring, "peer_call_plan", careless)
    with pytest.raises(AssertionError):
        for seed in range(300):
            _replay(4, calls=3, seed=seed)
