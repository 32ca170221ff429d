"""Head dims above 128 (the reference admits up to 256, sdp_utils.h:231-255, and its value tests run 256:
test/torch_ops/test_scaled_dot_product_attention.py:728-1285): the kernels that keep the stationary operand in
tensor memory, against the CPU oracle through the C ABI.

Tolerances: bf16 / fp16 outputs max-abs 2e-2 and mean-abs 2e-3, fp32 logsumexp 1e-5, gradients max(2e-2, 1e-2 |want|).
"""
import pytest
import torch

from oracle import sdpa_oracle as orc
from torch_mlu_b200 import ops

pytestmark = pytest.mark.gpu


def rand(shape, seed, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g).to(dtype)


@pytest.mark.parametrize("B,Hq,Hkv,Lq,Lk,D,causal", [
    (4, 2, 2, 512, 512, 256, True),      # the reference's own shape (test_...py:728-935), both mask settings
    (4, 2, 2, 512, 512, 256, False),
    (1, 2, 2, 1024, 2048, 256, True),    # from its sweep of lengths: Lq != Lk, bottom-right aligned mask
    (1, 2, 2, 2048, 512, 256, True),     # leading rows see no key
    (1, 1, 1, 128, 64, 256, False),      # one block
    (1, 1, 1, 1, 1, 256, True),          # minimum
    (2, 4, 2, 333, 777, 256, True),      # ragged lengths, GQA 2:1
    (1, 8, 1, 200, 130, 192, False),     # head_dim 192 (MQA): the last 64 columns are padding
    (2, 2, 2, 257, 255, 136, True),      # head_dim 136: padding inside a 64-column box
    (1, 2, 2, 130, 4100, 160, False),    # more blocks than ring slots several times over
])
def test_forward_head_dims_above_128(cuda_device, native_lib, B, Hq, Hkv, Lq, Lk, D, causal):
    dev = cuda_device
    q, k, v = rand((B, Hq, Lq, D), 1), rand((B, Hkv, Lk, D), 2), rand((B, Hkv, Lk, D), 3)
    out, lse = ops.gqa_prefill(q.to(dev), k.to(dev), v.to(dev), is_causal=causal)
    assert ops.device_status() == 0
    o_ref, l_ref = orc.cpu_sdpa_forward(q, k, v, causal=causal)
    orc.assert_close_bf16(out, o_ref, "out")
    orc.assert_close_lse(lse, l_ref)


def test_forward_head_dim_256_fp16_scale_and_layout(cuda_device, native_lib):
    dev = cuda_device
    B, H, L, D = 2, 3, 320, 256
    packed = rand((B, L, 3 * H * D), 5, torch.float16)
    q, k, v = (t.view(B, L, H, D).transpose(1, 2) for t in packed.chunk(3, dim=-1))
    qd, kd, vd = (t.view(B, L, H, D).transpose(1, 2) for t in packed.to(dev).chunk(3, dim=-1))
    for scale in (None, 0.01):
        out, lse = ops.gqa_prefill(qd, kd, vd, is_causal=True, scale=scale)
        o_ref, l_ref = orc.cpu_sdpa_forward(q, k, v, causal=True, scale=scale)
        orc.assert_close_bf16(out, o_ref, f"out scale={scale}")
        orc.assert_close_lse(lse, l_ref)


@pytest.mark.parametrize("lens,Hq,Hkv,D,causal", [
    ([100, 300, 257, 128], 4, 2, 256, True),
    ([1, 2, 255, 64, 65], 2, 2, 256, False),
    ([640, 130], 4, 1, 192, True),
])
def test_forward_packed_head_dims_above_128(cuda_device, native_lib, lens, Hq, Hkv, D, causal):
    dev = cuda_device
    total = sum(lens)
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    q, k, v = rand((total, Hq, D), 1), rand((total, Hkv, D), 2), rand((total, Hkv, D), 3)
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    out, lse, *_ = ops._flash_attention_forward(q.to(dev), k.to(dev), v.to(dev), cu_t, cu_t, max(lens), max(lens), 0.0, causal, False)
    assert ops.device_status() == 0
    o_ref, l_ref = orc.varlen_forward(q, k, v, cu, cu, causal=causal)
    orc.assert_close_bf16(out, o_ref, "out")
    orc.assert_close_lse(lse, l_ref)


def check_grads(got, want):
    for name, g, w in zip(("dq", "dk", "dv"), got, want):
        assert g.shape == w.shape, name
        orc.assert_close_grad_bf16(g, w, name)


@pytest.mark.parametrize("B,Hq,Hkv,Lq,Lk,D,causal", [
    (4, 2, 2, 512, 512, 256, True),      # the reference's backward shapes (test_...py:728-935)
    (4, 2, 2, 512, 512, 256, False),
    (1, 2, 2, 1024, 512, 256, True),     # leading rows see no key: their dq is 0
    (1, 2, 2, 512, 1024, 256, True),
    (1, 1, 1, 64, 128, 256, False),
    (1, 1, 1, 1, 1, 256, True),
    (2, 4, 2, 333, 777, 256, True),      # ragged lengths, GQA: dk / dv summed over two query heads
    (1, 8, 1, 200, 130, 192, False),     # MQA, padded head_dim
    (2, 2, 2, 257, 255, 136, True),
    (1, 2, 2, 130, 2100, 160, False),
])
def test_backward_head_dims_above_128(cuda_device, native_lib, B, Hq, Hkv, Lq, Lk, D, causal):
    dev = cuda_device
    q, k, v, dout = rand((B, Hq, Lq, D), 1), rand((B, Hkv, Lk, D), 2), rand((B, Hkv, Lk, D), 3), rand((B, Hq, Lq, D), 4)
    qd, kd, vd, dd = q.to(dev), k.to(dev), v.to(dev), dout.to(dev)
    out, lse = ops.gqa_prefill(qd, kd, vd, is_causal=causal)
    dq, dk, dv = ops._dense_backward(dd, qd, kd, vd, out, lse, causal, D ** -0.5)
    assert ops.device_status() == 0
    o_ref, l_ref = orc.cpu_sdpa_forward(q, k, v, causal=causal)
    check_grads((dq, dk, dv), orc.cpu_sdpa_backward(dout, q, k, v, o_ref, l_ref, causal=causal))
    # fixed summation order everywhere: the same call gives the same bits
    dq2, dk2, dv2 = ops._dense_backward(dd, qd, kd, vd, out, lse, causal, D ** -0.5)
    assert torch.equal(dq, dq2) and torch.equal(dk, dk2) and torch.equal(dv, dv2)


@pytest.mark.parametrize("lens,Hq,Hkv,D,causal", [
    ([100, 300, 257, 128], 4, 2, 256, True),
    ([1, 2, 255, 64, 65], 2, 2, 256, False),
    ([640, 130], 4, 1, 192, True),
])
def test_backward_packed_head_dims_above_128(cuda_device, native_lib, lens, Hq, Hkv, D, causal):
    dev = cuda_device
    total = sum(lens)
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    q, k, v, dout = rand((total, Hq, D), 1), rand((total, Hkv, D), 2), rand((total, Hkv, D), 3), rand((total, Hq, D), 4)
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    out, lse, seed, off, _ = ops._flash_attention_forward(qd, kd, vd, cu_t, cu_t, max(lens), max(lens), 0.0, causal, False)
    dq, dk, dv = ops._flash_attention_backward(dout.to(dev), qd, kd, vd, out, lse, cu_t, cu_t, max(lens), max(lens), 0.0, causal,
                                               seed, off)
    assert ops.device_status() == 0
    check_grads((dq, dk, dv), orc.varlen_backward(dout, q, k, v, cu, cu, causal=causal))


@pytest.mark.parametrize("B,Hq,Hkv,Lq,Lk,D,causal,p", [
    (4, 2, 2, 512, 512, 256, True, 0.22),    # the reference sweeps dropout 0.22 / 0.48 over head_dim 256 too (test_...py:938-946)
    (1, 2, 2, 512, 1024, 256, False, 0.48),
    (2, 4, 2, 200, 333, 192, True, 0.1),
])
def test_dropout_with_head_dims_above_128(cuda_device, native_lib, B, Hq, Hkv, Lq, Lk, D, causal, p):
    """Forward and backward with dropout against fp32 math on the CPU with the pattern rebuilt from the Philox pair
    (the restatement of the mask rule in the oracle)."""
    from torch_mlu_b200 import dropout
    dev = cuda_device
    q, k, v, dout = rand((B, Hq, Lq, D), 1), rand((B, Hkv, Lk, D), 2), rand((B, Hkv, Lk, D), 3), rand((B, Hq, Lq, D), 4)
    qd, kd, vd, dd = q.to(dev), k.to(dev), v.to(dev), dout.to(dev)
    seed, offset = 1234, 8
    keep = dropout.KeepMasks(seed, offset, p, B, Hq, Lq, Lk, dev, causal)
    sc = D ** -0.5
    out, lse = ops._dense_forward(qd, kd, vd, causal, sc, allow_gqa=True, kernel=1, keep=keep)
    dq, dk, dv = ops._dense_backward(dd, qd, kd, vd, out, lse, causal, sc, keep=keep)
    assert ops.device_status() == 0
    bits = orc.dropout_keep_mask(seed, offset, p, B, Hq, Lq, Lk)
    g = Hq // Hkv
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    scores = torch.einsum("bhqd,bhkd->bhqk", qf, kf.repeat_interleave(g, dim=1)) * sc
    if causal:
        scores = scores.masked_fill(orc.causal_mask_bottom_right(Lq, Lk), float("-inf"))
    l_ref = torch.logsumexp(scores, dim=-1)
    dead = torch.isinf(l_ref)
    attn = torch.softmax(scores, dim=-1).masked_fill(dead.unsqueeze(-1), 0.0).masked_fill(~bits, 0.0) / (1 - p)
    ref = torch.einsum("bhqk,bhkd->bhqd", attn, vf.repeat_interleave(g, dim=1))
    ref.backward(dout.float())
    orc.assert_close_bf16(out, ref.detach(), "out")
    orc.assert_close_lse(lse, l_ref.detach().masked_fill(dead, float("inf")))
    orc.assert_close_grad_bf16(dq, qf.grad, "dq")
    orc.assert_close_grad_bf16(dk, kf.grad, "dk")
    orc.assert_close_grad_bf16(dv, vf.grad, "dv")
