"""Launched by torchrun (one rank per GPU): ring prefill and batch x head sharding over NCCL,
each rank checking its own slice against the CPU oracle. Used by tests/test_ring_gpu.py when the
machine has at least two GPUs:
    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 tests/run_multigpu_ring.py
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from oracle import sdpa_oracle as orc  # noqa: E402
from torch_mlu_b200 import ring, sharding  # noqa: E402


def main():
    rank, local, world = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    g = torch.Generator().manual_seed(17)
    B, Hq, Hkv, Ls = 1, 8, 2, 512
    L = world * Ls
    q = torch.randn(B, Hq, L, 128, generator=g).bfloat16()
    k = torch.randn(B, Hkv, L, 128, generator=g).bfloat16()
    v = torch.randn(B, Hkv, L, 128, generator=g).bfloat16()
    sl = slice(rank * Ls, (rank + 1) * Ls)
    for causal in (False, True):
        out, lse = ring.ring_prefill(q[:, :, sl].to(dev), k[:, :, sl].to(dev), v[:, :, sl].to(dev), is_causal=causal)
        torch.cuda.synchronize()
        o_ref, l_ref = orc.cpu_sdpa_forward(q, k, v, causal=causal)
        orc.assert_close_bf16(out, o_ref[:, :, sl], f"ring out rank {rank} causal={causal}")
        orc.assert_close_lse(lse, l_ref[:, :, sl], max_abs=2e-5)
    take = lambda t: ring.zigzag_take(t, rank, world)
    out, lse = ring.ring_prefill(take(q).to(dev), take(k).to(dev), take(v).to(dev), is_causal=True, layout="zigzag")
    torch.cuda.synchronize()
    o_ref, l_ref = orc.cpu_sdpa_forward(q, k, v, causal=True)
    orc.assert_close_bf16(out, take(o_ref), f"zig-zag ring out rank {rank}")
    orc.assert_close_lse(lse, take(l_ref), max_abs=2e-5)
    # the same with SMs left to the hop's send/receive kernels: the grid size must not show in the result
    out2, lse2 = ring.ring_prefill(take(q).to(dev), take(k).to(dev), take(v).to(dev), is_causal=True, layout="zigzag",
                                   sm_margin=16)
    torch.cuda.synchronize()
    assert torch.equal(out, out2) and torch.equal(lse, lse2), f"sm_margin changed the ring's result on rank {rank}"
    # ... and with the slices pulled through CUDA IPC mappings by the copy engines, twice (the buffers are reused)
    for _ in range(2):
        out3, lse3 = ring.ring_prefill(take(q).to(dev), take(k).to(dev), take(v).to(dev), is_causal=True, layout="zigzag",
                                       exchange="peer")
        torch.cuda.synchronize()
        assert torch.equal(out, out3) and torch.equal(lse, lse3), f"the peer-copy exchange changed the result on rank {rank}"
    out4, lse4 = ring.ring_prefill(q[:, :, sl].to(dev), k[:, :, sl].to(dev), v[:, :, sl].to(dev), is_causal=False,
                                   exchange="peer")
    torch.cuda.synchronize()
    o_ref, l_ref = orc.cpu_sdpa_forward(q, k, v, causal=False)
    orc.assert_close_bf16(out4, o_ref[:, :, sl], f"peer-copy ring out rank {rank}")
    orc.assert_close_lse(lse4, l_ref[:, :, sl], max_abs=2e-5)
    # The transport's time limit: rank 0 starts a ring call that no other rank joins, so its first hop waits for a
    # counter nobody writes. The call must come back with an error after the limit, and everything after it must still
    # work (the waits are released, not left hanging).
    if rank == 0:
        try:
            ring.ring_prefill(take(q).to(dev), take(k).to(dev), take(v).to(dev), is_causal=True, layout="zigzag",
                              exchange="peer", peer_timeout_s=2.0)
            raise AssertionError("a ring call without partners returned normally")
        except RuntimeError as e:
            assert "did not complete within" in str(e), str(e)
    ring.release_peer_buffers()
    out, lse, _ = sharding.sdpa_batch_head_sharded(q.to(dev), k.to(dev), v.to(dev), is_causal=True)
    torch.cuda.synchronize()
    o_ref, l_ref = orc.cpu_sdpa_forward(q, k, v, causal=True)
    orc.assert_close_bf16(out, o_ref, f"sharded out rank {rank}")
    orc.assert_close_lse(lse, l_ref)
    dist.barrier()
    if rank == 0:
        print(f"multigpu ring ok: world {world}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
