"""HostPipeline: host tensors in and out over three streams give the same bits as the direct call."""
import pytest
import torch

from torch_mlu_b200 import ops
from torch_mlu_b200.host_pipeline import HostPipeline

pytestmark = pytest.mark.gpu


def test_pipelined_calls_match_direct_calls(cuda_device, native_lib):
    dev = cuda_device
    g = torch.Generator().manual_seed(31)
    B, H, L, D = 2, 4, 640, 128
    calls = []
    for _ in range(5):  # more calls than buffer sets, so slots are reused
        q, k, v = (torch.randn(B, H, L, D, generator=g).bfloat16().pin_memory() for _ in range(3))
        out = torch.empty(B, L, H, D, dtype=torch.bfloat16).pin_memory()
        lse = torch.empty(B, H, L, dtype=torch.float32).pin_memory()
        calls.append((q, k, v, out, lse))
    pipe = HostPipeline(dev, is_causal=True)
    for c in calls:
        pipe.submit(*c)
    pipe.wait()
    for q, k, v, out, lse in calls:
        o_ref, l_ref = ops.gqa_prefill(q.to(dev), k.to(dev), v.to(dev), is_causal=True)
        assert torch.equal(out, o_ref.transpose(1, 2).cpu())
        assert torch.equal(lse, l_ref.cpu())
    assert ops.device_status() == 0


def test_pageable_host_memory_is_refused(cuda_device, native_lib):
    pipe = HostPipeline(cuda_device, is_causal=False)
    t = torch.zeros(1, 1, 128, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="pinned"):
        pipe.submit(t, t, t, t, torch.zeros(1, 1, 128))
