"""The memory-efficient operators (attention.cpp:350-391, 510-600): same kernels
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
    with pytest.raises(RuntimeError, match="dtype and device of query"):
        ops._scaled_dot_product_efficient_attention(q, q, q, torch.zeros(1, 2, 128, 128, device=cuda_device), True)


def test_choice_prefers_flash_then_memory_efficient(cuda_device, native_lib):
    # short queries, head_dim 64: the default order (sdp_utils.cpp:8-50) tries flash first
    q64 = rand((1, 2, 64, 64), 1).to(cuda_device)
    assert sdp_choice._fused_sdp_choice(q64, q64, q64) == int(SDPBackend.FLASH_ATTENTION)
    q = rand((1, 2, 256, 128), 1).to(cuda_device)
    # inference with head_dim 128 puts the memory-efficient operator first; with it disabled, flash
    assert sdp_choice._fused_sdp_choice(q, q, q) == int(SDPBackend.EFFICIENT_ATTENTION)
    with backends.sdp_kernel(enable_flash=True, enable_math=True, enable_mem_efficient=False):
        assert sdp_choice._fused_sdp_choice(q, q, q) == int(SDPBackend.FLASH_ATTENTION)
    with backends.sdp_kernel(enable_flash=False, enable_math=True, enable_mem_efficient=True):
        assert sdp_choice._fused_sdp_choice(q, q, q) == int(SDPBackend.EFFICIENT_ATTENTION)
        out = sdp_choice.scaled_dot_product_attention(q, q, q, is_causal=True)
    ref = F.scaled_dot_product_attention(q.float().cpu(), q.float().cpu(), q.float().cpu(), is_causal=True)
    orc.assert_close_bf16(out, ref, "out through the memory efficient choice")


@pytest.mark.parametrize("mask_type,Lq,Lk", [(0, 300, 500), (1, 200, 456), (1, 456, 200), (2, 200, 456), (2, 384, 384)])
def test_efficient_attention_forward_backward_pair(cuda_device, native_lib, mask_type, Lq, Lk):
    """_efficient_attention_forward / _backward (attention.cpp:393-507, 579-727): [B, L, H, D] tensors, the three
    custom mask types of sdp_utils.h:32-37, logsumexp as [H, B*Lq]."""
    dev = cuda_device
    B, H, D = 2, 3, 128
    q, k, v, do = rand((B, Lq, H, D), 1), rand((B, Lk, H, D), 2), rand((B, Lk, H, D), 3), rand((B, Lq, H, D), 4)
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    out, lse, seed, off = ops._efficient_attention_forward(qd, kd, vd, None, None, None, None, 0.0, mask_type, True)
    assert tuple(out.shape) == (B, H, Lq, D) and tuple(lse.shape) == (H, B * Lq)
    out_blhd = out.transpose(1, 2)
    dq, dk, dv, dbias = ops._efficient_attention_backward(do.to(dev), qd, kd, vd, None, out_blhd, None, None, Lk, Lq, lse, 0.0,
                                                         seed, off, mask_type, False)
    assert ops.device_status() == 0 and dbias.numel() == 0
    assert tuple(dq.shape) == (B, Lq, H, D) and tuple(dk.shape) == (B, Lk, H, D) and tuple(dv.shape) == (B, Lk, H, D)
    qf, kf, vf = (t.float().transpose(1, 2).detach().requires_grad_(True) for t in (q, k, v))
    scores = torch.einsum("bhqd,bhkd->bhqk", qf, kf) / D ** 0.5
    if mask_type == 1:
        scores = scores.masked_fill(torch.ones(Lq, Lk, dtype=torch.bool).triu(1), float("-inf"))
    elif mask_type == 2:
        scores = scores.masked_fill(orc.causal_mask_bottom_right(Lq, Lk), float("-inf"))
    l_ref = torch.logsumexp(scores, dim=-1)
    dead = torch.isinf(l_ref)
    attn = torch.softmax(scores, dim=-1).masked_fill(dead.unsqueeze(-1), 0.0)
    ref = torch.einsum("bhqk,bhkd->bhqd", attn, vf)
    ref.backward(do.float().transpose(1, 2))
    orc.assert_close_bf16(out, ref.detach(), "out")
    orc.assert_close_lse(lse.view(H, B, Lq).permute(1, 0, 2), l_ref.detach().masked_fill(dead, float("inf")))
    orc.assert_close_grad_bf16(dq.transpose(1, 2), qf.grad, "dq")
    orc.assert_close_grad_bf16(dk.transpose(1, 2), kf.grad, "dk")
    orc.assert_close_grad_bf16(dv.transpose(1, 2), vf.grad, "dv")


def test_efficient_attention_with_cu_seqlens(cuda_device, native_lib):
    """cu_seqlens index the flattened B*L token axis (attention.cpp:435-470): two sequences of 200 and 256 tokens
    inside a [2, 256] token grid; the tokens after the last offset belong to no sequence."""
    dev = cuda_device
    B, L, H, D = 2, 256, 2, 64
    q, k, v, do = (rand((B, L, H, D), s) for s in (1, 2, 3, 4))
    cu = [0, 200, 456]
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    out, lse, seed, off = ops._efficient_attention_forward(qd, kd, vd, None, cu_t, cu_t, 256, 0.0, 1, True)
    dq, dk, dv, _ = ops._efficient_attention_backward(do.to(dev), qd, kd, vd, None, out.transpose(1, 2), cu_t, cu_t, 256, 256, lse,
                                                     0.0, seed, off, 1, False)
    assert ops.device_status() == 0
    flat = lambda x: x.reshape(B * L, H, D)
    o_ref, l_ref = orc.varlen_forward(flat(q), flat(k), flat(v), cu, cu, causal=True)
    n = cu[-1]
    orc.assert_close_bf16(flat(out.transpose(1, 2))[:n], o_ref, "out")
    orc.assert_close_lse(lse[:, :n], l_ref)
    want = orc.varlen_backward(flat(do)[:n], flat(q)[:n], flat(k)[:n], flat(v)[:n], cu, cu, causal=True)
    for name, g, w in zip(("dq", "dk", "dv"), (dq, dk, dv), want):
        orc.assert_close_grad_bf16(flat(g)[:n], w, name)


def test_efficient_attention_with_dropout(cuda_device, native_lib):
    """The reference sweeps dropout_p over the memory-efficient operator too (test_...py:1379-1402). The pattern is
    rebuilt from the returned Philox pair with the CPU restatement of the mask rule."""
    dev = cuda_device
    B, H, L, D, p = 2, 2, 320, 128, 0.48
    q, k, v = (rand((B, H, L, D), s) for s in (1, 2, 3))
    do = torch.rand((B, H, L, D), generator=torch.Generator().manual_seed(4)).bfloat16()
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    out, lse, seed, off = ops._scaled_dot_product_efficient_attention(qd, kd, vd, None, True, p, True)
    dq, dk, dv, _ = ops._scaled_dot_product_efficient_attention_backward(do.to(dev), qd, kd, vd, None, out, lse, seed, off, p,
                                                                        [True, True, True, False], True)
    assert ops.device_status() == 0
    keep = orc.dropout_keep_mask(int(seed), int(off), p, B, H, L, L)
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    scores = torch.einsum("bhqd,bhkd->bhqk", qf, kf) / D ** 0.5
    scores = scores.masked_fill(torch.ones(L, L, dtype=torch.bool).triu(1), float("-inf"))
    attn = torch.softmax(scores, dim=-1).masked_fill(~keep, 0.0) / (1 - p)
    ref = torch.einsum("bhqk,bhkd->bhqd", attn, vf)
    ref.backward(do.float())
    orc.assert_close_bf16(out, ref.detach(), "out")
    orc.assert_close_grad_bf16(dq, qf.grad, "dq")
    orc.assert_close_grad_bf16(dk, kf.grad, "dk")
    orc.assert_close_grad_bf16(dv, vf.grad, "dv")


@pytest.mark.parametrize("Lq,Lk", [(200, 456), (456, 200)])
def test_efficient_attention_with_dropout_and_unequal_lengths(cuda_device, native_lib, Lq, Lk):
    """Top-left causal mask with Lq != Lk and dropout: the operator is made of one or two kernel calls, each with
    its own pattern from the one Philox pair (the second call, rows past Lk, on the stream with bit 62 of the
    offset set)."""
    dev = cuda_device
    B, H, D, p = 1, 2, 128, 0.22
    q, k, v = rand((B, H, Lq, D), 1), rand((B, H, Lk, D), 2), rand((B, H, Lk, D), 3)
    do = torch.rand((B, H, Lq, D), generator=torch.Generator().manual_seed(4)).bfloat16()
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    out, lse, seed, off = ops._scaled_dot_product_efficient_attention(qd, kd, vd, None, True, p, True)
    dq, dk, dv, _ = ops._scaled_dot_product_efficient_attention_backward(do.to(dev), qd, kd, vd, None, out, lse, seed, off, p,
                                                                        [True, True, True, False], True)
    assert ops.device_status() == 0
    s0, o0 = int(seed), int(off)
    keep = torch.zeros(B, H, Lq, Lk, dtype=torch.bool)
    if Lq < Lk:
        keep[..., :Lq] = orc.dropout_keep_mask(s0, o0, p, B, H, Lq, Lq)       # keys past Lq are hidden anyway
    else:
        keep[:, :, :Lk] = orc.dropout_keep_mask(s0, o0, p, B, H, Lk, Lk)
        keep[:, :, Lk:] = orc.dropout_keep_mask(s0, o0 ^ (1 << 62), p, B, H, Lq - Lk, Lk)

    def run(dtype):
        qf, kf, vf = (t.to(dtype).requires_grad_(True) for t in (q, k, v))
        scores = torch.einsum("bhqd,bhkd->bhqk", qf, kf) / D ** 0.5
        scores = scores.masked_fill(torch.ones(Lq, Lk, dtype=torch.bool).triu(1), float("-inf"))
        attn = torch.softmax(scores, dim=-1).masked_fill(~keep, 0.0) / (1 - p)
        ref = torch.einsum("bhqk,bhkd->bhqd", attn, vf)
        ref.backward(do.to(dtype))
        return ref.detach(), qf.grad, kf.grad, vf.grad

    # gradients by the reference suite's own rule (test_...py:1077-1110): dV sums hundreds of queries per key here
    true, lowp = run(torch.float32), run(torch.bfloat16)
    orc.assert_close_bf16(out, true[0], "out")
    orc.assert_close_reference_rule(dq, true[1], lowp[1], "dq", fudge=4)
    orc.assert_close_reference_rule(dk, true[2], lowp[2], "dk")
    orc.assert_close_reference_rule(dv, true[3], lowp[3], "dv")


def _bias_reference(q, k, v, bias, do, causal_top_left, dtype=torch.float32):
    qf, kf, vf, bf = (t.to(dtype).detach().requires_grad_(True) for t in (q, k, v, bias))
    scores = torch.einsum("bhqd,bhkd->bhqk", qf, kf) * (q.shape[-1] ** -0.5) + bf
    if causal_top_left:
        scores = scores.masked_fill(torch.ones(q.shape[2], k.shape[2], dtype=torch.bool).triu(1), float("-inf"))
    out = torch.einsum("bhqk,bhkd->bhqd", torch.softmax(scores, dim=-1), vf)
    out.backward(do.to(dtype))
    return out.detach(), torch.logsumexp(scores.detach().float(), dim=-1), qf.grad, kf.grad, vf.grad, bf.grad


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("Lq,Lk,D,causal,bias_shape", [
    (256, 256, 128, False, (2, 3, 256, 256)),    # full bias, read in place
    (200, 333, 128, False, (1, 3, 200, 333)),    # batch broadcast, ragged key length: padded copy
    (300, 300, 64, True, (2, 1, 300, 300)),      # head broadcast with the causal mask
    (130, 257, 128, True, (1, 1, 1, 257)),       # one bias row for every query; top-left causal with Lq < Lk
    (257, 130, 96, True, (2, 3, 257, 130)),      # top-left causal with Lq > Lk: two kernel calls
])
def test_attn_bias_forward_and_backward(cuda_device, native_lib, dtype, Lq, Lk, D, causal, bias_shape):
    """Additive bias through the memory-efficient operators, as the reference tests exercise it (a random
    attn_mask in the low-precision dtype next to q, k, v; test_...py:1445-1511, 1800-1901): output, log_sumexp and
    all four gradients against autograd through the fp32 math, held to that suite's own tolerance rule, and to
    the fixed tolerances where values are of order one."""
    dev = cuda_device
    B, H = 2, 3
    g = torch.Generator().manual_seed(7)
    q, k, v = (torch.randn(s, generator=g).to(dtype) for s in ((B, H, Lq, D), (B, H, Lk, D), (B, H, Lk, D)))
    bias = torch.rand(bias_shape, generator=g).to(dtype)
    do = torch.rand((B, H, Lq, D), generator=g).to(dtype)
    qd, kd, vd, bd = q.to(dev), k.to(dev), v.to(dev), bias.to(dev)
    out, lse, seed, off = ops._scaled_dot_product_efficient_attention(qd, kd, vd, bd, True, 0.0, causal)
    dq, dk, dv, db = ops._scaled_dot_product_efficient_attention_backward(do.to(dev), qd, kd, vd, bd, out, lse, seed, off, 0.0,
                                                                         [True, True, True, True], causal)
    assert ops.device_status() == 0 and tuple(db.shape) == tuple(bias_shape)
    true = _bias_reference(q, k, v, bias, do, causal)
    lowp = _bias_reference(q, k, v, bias, do, causal, dtype)
    orc.assert_close_bf16(out, true[0], "out")
    orc.assert_close_lse(lse, true[1])
    for name, got, i, fudge in (("dq", dq, 2, 4), ("dk", dk, 3, 2), ("dv", dv, 4, 2), ("dbias", db, 5, 4)):
        orc.assert_close_reference_rule(got, true[i], lowp[i], name, fudge=fudge)
    for name, got, i in (("dq", dq, 2), ("dk", dk, 3), ("dv", dv, 4)):
        orc.assert_close_grad_bf16(got, true[i], name)
    # without asking for it there is no bias gradient
    *_, none = ops._scaled_dot_product_efficient_attention_backward(do.to(dev), qd, kd, vd, bd, out, lse, seed, off, 0.0,
                                                                    [True, True, True, False], causal)
    assert none.numel() == 0


def test_attn_bias_of_minus_infinity_masks_keys(cuda_device, native_lib):
    """A bias of -inf hides a key (the boolean attn_mask of F.scaled_dot_product_attention arrives that way)."""
    dev = cuda_device
    B, H, L, D = 1, 2, 256, 128
    q, k, v = (rand((B, H, L, D), s) for s in (1, 2, 3))
    bias = torch.zeros(1, 1, L, L)
    bias[..., 100:180] = float("-inf")
    out, lse, _, _ = ops._scaled_dot_product_efficient_attention(q.to(dev), k.to(dev), v.to(dev), bias.bfloat16().to(dev), True)
    ref = F.scaled_dot_product_attention(q.float(), k.float(), v.float(), attn_mask=bias)
    orc.assert_close_bf16(out, ref, "out")


def test_efficient_attention_pair_with_bias_and_dropout_with_bias(cuda_device, native_lib):
    dev = cuda_device
    B, H, L, D = 1, 2, 256, 128
    q, k, v, do = (rand((B, L, H, D), s) for s in (1, 2, 3, 4))
    bias = torch.rand((B, H, L, L), generator=torch.Generator().manual_seed(5)).bfloat16()
    qd, kd, vd, bd = q.to(dev), k.to(dev), v.to(dev), bias.to(dev)
    out, lse, seed, off = ops._efficient_attention_forward(qd, kd, vd, bd, None, None, None, 0.0, 2, True)
    dq, dk, dv, db = ops._efficient_attention_backward(do.to(dev), qd, kd, vd, bd, out.transpose(1, 2), None, None, L, L, lse, 0.0,
                                                      seed, off, 2, True)
    t = lambda x: x.transpose(1, 2)
    true = _bias_reference(t(q), t(k), t(v), bias, t(do), True)
    orc.assert_close_bf16(out, true[0], "out")
    orc.assert_close_grad_bf16(t(dq), true[2], "dq")
    orc.assert_close_grad_bf16(t(dk), true[3], "dk")
    orc.assert_close_grad_bf16(t(dv), true[4], "dv")
    orc.assert_close_grad_bf16(db, true[5], "dbias")
    # bias together with dropout: the pattern is rebuilt from the returned Philox pair
    p = 0.22
    q4, k4, v4, do4 = t(q), t(k), t(v), t(do)
    out, lse, seed, off = ops._scaled_dot_product_efficient_attention(q4.to(dev), k4.to(dev), v4.to(dev), bd, True, p, False)
    dq, dk, dv, db = ops._scaled_dot_product_efficient_attention_backward(do4.to(dev), q4.to(dev), k4.to(dev), v4.to(dev), bd, out,
                                                                         lse, seed, off, p, [True, True, True, True], False)
    keep = orc.dropout_keep_mask(int(seed), int(off), p, B, H, L, L)
    qf, kf, vf, bf = (x.float().detach().requires_grad_(True) for x in (q4, k4, v4, bias))
    attn = torch.softmax(torch.einsum("bhqd,bhkd->bhqk", qf, kf) * D ** -0.5 + bf, dim=-1).masked_fill(~keep, 0.0) / (1 - p)
    ref = torch.einsum("bhqk,bhkd->bhqd", attn, vf)
    ref.backward(do4.float())
    orc.assert_close_bf16(out, ref.detach(), "out")
    for name, got, want in (("dq", dq, qf.grad), ("dk", dk, kf.grad), ("dv", dv, vf.grad), ("dbias", db, bf.grad)):
        orc.assert_close_grad_bf16(got, want, name)


def test_choice_routes_an_attn_mask_to_the_memory_efficient_kernels_with_autograd(cuda_device, native_lib):
    """scaled_dot_product_attention with an attn_mask: flash refuses it, the memory-efficient backend takes it as
    additive bias (boolean masks become 0 / -inf), and gradients flow to q, k, v and a floating-point mask."""
    dev = cuda_device
    B, H, L, D = 2, 2, 192, 128
    q, k, v, do = (rand((B, H, L, D), s) for s in (1, 2, 3, 4))
    fmask = torch.rand((B, 1, L, L), generator=torch.Generator().manual_seed(9)).bfloat16()
    qd, kd, vd, md = (t.to(dev).requires_grad_(True) for t in (q, k, v, fmask))
    assert sdp_choice._fused_sdp_choice(qd, kd, vd, md) == int(SDPBackend.EFFICIENT_ATTENTION)
    out = sdp_choice.scaled_dot_product_attention(qd, kd, vd, attn_mask=md)
    out.backward(do.to(dev))
    qf, kf, vf, mf = (t.float().requires_grad_(True) for t in (q, k, v, fmask))
    ref = F.scaled_dot_product_attention(qf, kf, vf, attn_mask=mf)
    ref.backward(do.float())
    orc.assert_close_bf16(out, ref.detach(), "out")
    for name, got, want in (("dq", qd.grad, qf.grad), ("dk", kd.grad, kf.grad), ("dv", vd.grad, vf.grad),
                            ("dmask", md.grad, mf.grad)):
        assert got.shape == want.shape
        orc.assert_close_grad_bf16(got, want, name)
    bmask = torch.rand((L, L), generator=torch.Generator().manual_seed(10)) > 0.3
    bmask[:, 0] = True  # no empty rows
    out = sdp_choice.scaled_dot_product_attention(q.to(dev), k.to(dev), v.to(dev), attn_mask=bmask.to(dev))
    ref = F.scaled_dot_product_attention(q.float(), k.float(), v.float(), attn_mask=bmask)
    orc.assert_close_bf16(out, ref, "out with a boolean mask")


@pytest.mark.parametrize("Lq,Lk,causal", [(256, 256, True), (200, 333, False)])
def test_backward_with_a_transposed_bias_copy_gives_the_same_gradients(cuda_device, native_lib, Lq, Lk, causal):
    """The optional bias_t of the C ABI (the bias with keys and queries exchanged, read 16 bytes at a time by the
    dK/dV kernel) against the same call without it: bit-identical gradients."""
    dev = cuda_device
    B, H, D = 2, 2, 128
    q, k, v, do = rand((B, H, Lq, D), 1).to(dev), rand((B, H, Lk, D), 2).to(dev), rand((B, H, Lk, D), 3).to(dev), rand((B, H, Lq, D), 4).to(dev)
    bias = ops._prepare_bias(torch.rand((B, 1, Lq, Lk), generator=torch.Generator().manual_seed(3)).bfloat16().to(dev), q, k)
    sc = ops.calculate_scale(q, None)
    out, lse = ops._dense_forward(q, k, v, causal, sc, allow_gqa=False, bias=bias)
    plain = ops._dense_backward(do, q, k, v, out, lse, causal, sc, bias=bias, bias_t=False)
    bias_t = ops._transposed_bias(bias)
    assert bias_t is not None and tuple(bias_t.shape) == (B, H, Lk, Lq) and bias_t.stride(1) == 0   # heads stay broadcast
    assert torch.equal(bias_t, bias.transpose(2, 3))
    fast = ops._dense_backward(do, q, k, v, out, lse, causal, sc, bias=bias, bias_t=bias_t)
    assert ops.device_status() == 0
    for a, b in zip(plain, fast):
        assert torch.equal(a, b)
    assert ops._transposed_bias(bias[:, :, :1].expand(B, H, Lq, Lk)) is None   # no query dependence: nothing to copy
