"""sdpa_b200_decode_static: split-KV decode for callers that must not allocate device memory
(code running inside an allocator or memory-pool callback, or a server that froze its memory
plan at start-up). The split partials live in a fixed array inside the library, so the call
takes only inputs and outputs. Checked here against the ordinary workspace-based entry point,
through the C ABI, on two consecutive calls that share (and overwrite) the same static array.
Collected last on purpose: a run that stops at the first failure has already seen every other test.
"""
import ctypes

import pytest
import torch

from oracle import sdpa_oracle as orc
from torch_mlu_b200 import _cabi, ops

pytestmark = pytest.mark.gpu


def rand(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g).bfloat16()


def decode_params(q, k, v, out, lse, num_splits):
    p = ops._dense_params(q, k, v, out, lse, False, ops.calculate_scale(q, None), _cabi.KERNEL_DECODE, num_splits)
    return p


def run_static(lib, q, k, v, num_splits):
    """The new entry point: caller-owned out/lse, no workspace argument at all."""
    B, Hq = q.shape[0], q.shape[1]
    out = torch.full((B, Hq, 1, q.shape[-1]), float("nan"), dtype=torch.bfloat16, device=q.device)
    lse = torch.full((B, Hq, 1), float("nan"), dtype=torch.float32, device=q.device)
    p = decode_params(q, k, v, out, lse, num_splits)
    st = lib.sdpa_b200_decode_static(ctypes.byref(p), torch.cuda.current_stream().cuda_stream)
    _cabi.check(st, "sdpa_b200_decode_static")
    return out, lse


def test_static_scratch_decode_matches_workspace_decode_twice(cuda_device, native_lib):
    dev = cuda_device
    lib = native_lib
    # two different problems back to back: the second starts from the first one's leftovers
    # (the head_dim 64 case runs the other kernel instance, whose partial slots are half as wide)
    cases = [((4, 32, 8, 6000), 128, 8, 1), ((2, 8, 2, 1500), 128, 5, 2), ((3, 16, 4, 3000), 64, 6, 4),
             ((4, 32, 8, 6000), 128, 8, 3)]
    for (B, Hq, Hkv, Lk), D, splits, seed in cases:
        q = rand((B, Hq, 1, D), seed).to(dev)
        k = rand((B, Hkv, Lk, D), seed + 10).to(dev)
        v = rand((B, Hkv, Lk, D), seed + 20).to(dev)
        before = torch.cuda.memory_allocated(dev)
        out_s, lse_s = run_static(lib, q, k, v, splits)
        # only the two output tensors this test created were allocated around the call
        assert torch.cuda.memory_allocated(dev) - before <= out_s.numel() * 2 + lse_s.numel() * 4 + 1024
        out_w, lse_w = ops.decode_attention(q, k, v, num_splits=splits)
        torch.cuda.synchronize()
        # same kernels, same split count: the two entry points agree to the bit, and both meet
        # the oracle at the usual tolerances (bf16 out 2e-2 / 2e-3, fp32 lse 1e-5)
        assert torch.equal(out_s, out_w) and torch.equal(lse_s, lse_w)
        o_ref, l_ref = orc.cpu_sdpa_forward(q.cpu(), k.cpu(), v.cpu())
        orc.assert_close_bf16(out_s, o_ref, "static out")
        orc.assert_close_lse(lse_s, l_ref, "static lse")


def test_static_scratch_decode_refuses_oversized_requests(cuda_device, native_lib):
    dev = cuda_device
    lib = native_lib
    # 64 x 32 heads x 64 splits x 516 B = 67.6 MB of partials > the 16 MiB built in
    B, Hq, Hkv, Lk = 64, 32, 8, 4096
    q = rand((B, Hq, 1, 128), 1).to(dev)
    k = torch.zeros((B, Hkv, Lk, 128), dtype=torch.bfloat16, device=dev)
    out = torch.empty((B, Hq, 1, 128), dtype=torch.bfloat16, device=dev)
    lse = torch.empty((B, Hq, 1), dtype=torch.float32, device=dev)
    p = decode_params(q, k, k, out, lse, 64)
    st = lib.sdpa_b200_decode_static(ctypes.byref(p), torch.cuda.current_stream().cuda_stream)
    assert st == _cabi.INVALID_ARG
    msg = lib.sdpa_b200_last_error().decode()
    assert "more than the" in msg and str(_cabi.STATIC_SCRATCH_BYTES) in msg
    # prefill-shaped input is not this entry point's business
    q4 = rand((1, 8, 4, 128), 2).to(dev)
    p = decode_params(q4, k[:1], k[:1], out, lse, 1)
    assert lib.sdpa_b200_decode_static(ctypes.byref(p), None) == _cabi.UNSUPPORTED
    # a head dim the streaming kernels are not built for is refused, not run in the 128-column instance
    q96, k96 = rand((2, 8, 1, 96), 3).to(dev), rand((2, 2, 512, 96), 4).to(dev)
    out96 = torch.full((2, 8, 1, 96), float("nan"), dtype=torch.bfloat16, device=dev)
    p = decode_params(q96, k96, k96, out96, lse, 2)
    assert lib.sdpa_b200_decode_static(ctypes.byref(p), None) == _cabi.UNSUPPORTED
    torch.cuda.synchronize()
    assert torch.isnan(out96).all()
