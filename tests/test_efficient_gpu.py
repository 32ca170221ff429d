"""The bias-free subset of the memory-efficient operators (attention.cpp:350-391, 510-600): same kernels
as the flash operators, but a causal mask aligned to the TOP-LEFT corner (sdp_utils.h:32-37). torch's CPU
scaled_dot_product_attention uses the same convention, so it is the fp32 reference here (forward and, by
autograd, backward). Tolerances as everywhere: out / grads max-abs 2e-2, mean-abs 2e-3; lse 1e-5."""
import pytest
import torch
import torch.nn.functional as F

from oracle import sdpa_oracle as orc
from torch_mlu_b200 import backends, ops, sdp_choice
from torch_mlu_b200.backends import SDPBackend

pytestmark = pytest.mark.gpu


def rand(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g).bfloat16()


@pytest.mark.parametrize("Lq,Lk,causal", [(384, 384, True), (200, 456, True), (456, 200, True), (300, 500, False)])
def test_efficient_forward_backward_top_left_causal(cuda_device, native_lib, Lq, Lk, causal):
    dev = cuda_device
    B, H, D = 2, 4, 128
    q, k, v, do = rand((B, H, Lq, D), 1), rand((B, H, Lk, D), 2), rand((B, H, Lk, D), 3), rand((B, H, Lq, D), 4)
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    out, lse, seed, off = ops._scaled_dot_product_efficient_attention(qd, kd, vd, None, True, 0.0, causal)
    assert tuple(lse.shape) == (B, H, Lq) and seed.numel() == 0
    dq, dk, dv, dbias = ops._scaled_dot_product_efficient_attention_backward(
        do.to(dev), qd, kd, vd, None, out, lse, seed, off, 0.0, [True, True, True, False], causal)
    assert ops.device_status() == 0 and dbias.numel() == 0
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    ref = F.scaled_dot_product_attention(qf, kf, vf, is_causal=causal)  # CPU: top-left causal
    ref.backward(do.float())
    orc.assert_close_bf16(out, ref.detach(), "out")
    scores = torch.einsum("bhqd,bhkd->bhqk", q.float(), k.float()) / D ** 0.5
    if causal:
        scores = scores.masked_fill(torch.ones(Lq, Lk, dtype=torch.bool).triu(1), float("-inf"))
    orc.assert_close_lse(lse, torch.logsumexp(scores, dim=-1))
    orc.assert_close_grad_bf16(dq, qf.grad, "dq")
    orc.assert_close_grad_bf16(dk, kf.grad, "dk")
    orc.assert_close_grad_bf16(dv, vf.grad, "dv")


def test_efficient_without_log_sumexp_and_with_bias(cuda_device, native_lib):
    q = rand((1, 2, 128, 128), 1).to(cuda_device)
    out, lse, _, _ = ops._scaled_dot_product_efficient_attention(q, q, q, None, False)
    assert lse.numel() == 0 and out.shape == q.shape
    with pytest.raises(RuntimeError, match="attn_bias is not supported"):
        ops._scaled_dot_product_efficient_attention(q, q, q, torch.zeros(1, 2, 128, 128, device=cuda_device), True)


def test_choice_prefers_flash_then_memory_efficient(cuda_device, native_lib):
    q = rand((1, 2, 256, 128), 1).to(cuda_device)
    assert sdp_choice._fused_sdp_choice(q, q, q) == int(SDPBackend.FLASH_ATTENTION)
    with backends.sdp_kernel(enable_flash=False, enable_math=True, enable_mem_efficient=True):
        assert sdp_choice._fused_sdp_choice(q, q, q) == int(SDPBackend.EFFICIENT_ATTENTION)
        out = sdp_choice.scaled_dot_product_attention(q, q, q, is_causal=True)
    ref = F.scaled_dot_product_attention(q.float().cpu(), q.float().cpu(), q.float().cpu(), is_causal=True)
    orc.assert_close_bf16(out, ref, "out through the memory efficient choice")
