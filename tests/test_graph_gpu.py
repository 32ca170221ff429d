"""The C-ABI calls enqueue work on the caller's stream and nothing else (no allocation, no hidden
synchronisation), so forward + backward can be captured in a CUDA graph and replayed on new data."""
import pytest
import torch

from torch_mlu_b200 import ops

pytestmark = pytest.mark.gpu


def test_forward_backward_replay_in_a_cuda_graph(cuda_device, native_lib):
    dev = cuda_device
    g = torch.Generator().manual_seed(41)
    B, H, L, D = 2, 4, 768, 128
    scale = D ** -0.5
    make = lambda: torch.randn(B, H, L, D, generator=g).bfloat16().to(dev)
    q, k, v, do = make(), make(), make(), make()
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):  # warm-up outside capture: library handles, kernel attributes
        out, lse = ops.gqa_prefill(q, k, v, is_causal=True)
        ops._dense_backward(do, q, k, v, out, lse, True, scale)
    torch.cuda.current_stream(dev).wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out, lse = ops.gqa_prefill(q, k, v, is_causal=True)
        dq, dk, dv = ops._dense_backward(do, q, k, v, out, lse, True, scale)
    for _ in range(2):  # replay twice on fresh inputs: the persistent kernel's unit counter is reset by a graph node too
        for t in (q, k, v, do):
            t.copy_(torch.randn(B, H, L, D, generator=g).bfloat16())
        graph.replay()
        torch.cuda.synchronize()
        got = [t.clone() for t in (out, lse, dq, dk, dv)]
        o2, l2 = ops.gqa_prefill(q, k, v, is_causal=True)
        want = [o2, l2, *ops._dense_backward(do, q, k, v, o2, l2, True, scale)]
        assert ops.device_status() == 0
        for a, b in zip(got, want):
            assert torch.equal(a, b)
