"""GPU side of ring / context-parallel prefill: the logsumexp fold kernel against its torch
statement, and a one-GPU emulation of a 4-slice ring (the slices visit in ring order) against
full attention from the CPU oracle. The real multi-GPU exchange needs more than one device."""
import pytest
import torch

from oracle import sdpa_oracle as orc
from torch_mlu_b200 import ops, ring

pytestmark = pytest.mark.gpu


def rand(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g).bfloat16()


def test_merge_kernel_matches_torch_statement(cuda_device, native_lib):
    dev = cuda_device
    B, H, L = 2, 3, 200
    o_acc = torch.randn(B, H, L, 128, device=dev)
    lse_acc = torch.randn(B, H, L, device=dev) * 3
    lse_acc[0, 0, :5] = float("-inf")
    o_part = rand((B, L, H, 128), 1).to(dev).transpose(1, 2)  # strided view, as the forward returns
    lse_part = torch.randn(B, H, L, device=dev) * 3
    lse_part[0, 0, 3:8] = float("inf")
    want_o, want_l = o_acc.clone(), lse_acc.clone()
    ring.merge_partial_reference(want_o, want_l, o_part, lse_part)
    ring.merge_partial(o_acc, lse_acc, o_part, lse_part)
    assert torch.equal(torch.isinf(lse_acc), torch.isinf(want_l))
    fin = torch.isfinite(want_l)
    assert (lse_acc[fin] - want_l[fin]).abs().max() < 2e-6
    assert (o_acc - want_o).abs().max() < 1e-5


@pytest.mark.parametrize("causal", [False, True])
def test_ring_order_emulated_on_one_gpu(cuda_device, native_lib, causal):
    dev = cuda_device
    world, B, Hq, Hkv, Ls = 4, 1, 4, 2, 256
    L = world * Ls
    q, k, v = rand((B, Hq, L, 128), 1), rand((B, Hkv, L, 128), 2), rand((B, Hkv, L, 128), 3)
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    o_ref, l_ref = orc.cpu_sdpa_forward(q, k, v, causal=causal)
    for rank in range(world):
        sl = slice(rank * Ls, (rank + 1) * Ls)
        o_acc = torch.empty((B, Hq, Ls, 128), dtype=torch.float32, device=dev)
        lse_acc = torch.full((B, Hq, Ls), float("-inf"), dtype=torch.float32, device=dev)
        for step in range(world):
            src = (rank - step) % world
            if causal and src > rank:
                continue
            ks = slice(src * Ls, (src + 1) * Ls)
            o_part, lse_part = ops.gqa_prefill(qd[:, :, sl], kd[:, :, ks], vd[:, :, ks], is_causal=causal and src == rank)
            ring.merge_partial(o_acc, lse_acc, o_part, lse_part)
        orc.assert_close_bf16(o_acc.bfloat16(), o_ref[:, :, sl], f"out rank {rank}")
        orc.assert_close_lse(lse_acc, l_ref[:, :, sl], max_abs=2e-5)


def test_ring_and_sharding_over_nccl_when_two_gpus_are_present(cuda_device, native_lib):
    """Real exchange over NCCL, one process per GPU (plain peer transfers: NVLS off)."""
    import os
    import subprocess
    import sys
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    world = 2 if n < 4 else 4
    script = os.path.join(os.path.dirname(os.path.abspath(__file__)), "run_multigpu_ring.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                        "--master-addr", "127.0.0.1", "--master-port", "29533", script], capture_output=True, text=True,
                       env=env, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "multigpu ring ok" in r.stdout
