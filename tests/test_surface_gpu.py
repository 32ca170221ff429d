"""Operator-surface details a drop-in caller can see, on the GPU:

* ``_efficient_attention_forward/_backward`` with dropout, and with a bias together with cu_seqlens - the reference
  hands both to its kernel (attention.cpp:393-507, 579-727; tests test_scaled_dot_product_attention.py:1372-1952);
* the logsumexp of ``_scaled_dot_product_flash_attention`` padded to a multiple of 16 rows
  (FlashAttention_internal.cpp:261-265) and cut back by the backward (:374-375);
* ``return_debug_mask`` for packed tensors through the registered operator (attention.cpp:178-196);
* the backward takes the keep-masks its forward left instead of drawing them again, with the same result;
* the time-out path: a kernel whose bounded wait runs out reports DEVICE_TIMEOUT and the context stays usable.

Tolerances: bf16 outputs max-abs 2e-2 / mean-abs 2e-3, gradients max(2e-2, 1e-2 |want|), fp32 logsumexp 1e-5.
"""
import ctypes

import pytest
import torch

from oracle import sdpa_oracle as orc
from torch_mlu_b200 import _cabi, dropout, ops

pytestmark = pytest.mark.gpu


def rand(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g).bfloat16()


def fp32_attention(q, k, v, do, *, visible=None, bias=None, keep=None, p=0.0):
    """softmax(scale q k^T + bias) over the visible keys, dropout by `keep`, and its gradients, in fp32 on the CPU.
    q, k, v, do: [B, H, L, D]. Returns (out, lse, dq, dk, dv, ds) with ds the gradient of the scores (= of the bias)."""
    D = q.size(-1)
    qf, kf, vf = (t.float().detach().requires_grad_(True) for t in (q, k, v))
    scores = torch.einsum("bhqd,bhkd->bhqk", qf, kf) * D ** -0.5
    if bias is not None:
        bf = bias.float().detach().expand_as(scores).clone().requires_grad_(True)
        scores = scores + bf
    if visible is not None:
        scores = scores.masked_fill(~visible, float("-inf"))
    lse = torch.logsumexp(scores, dim=-1)
    dead = torch.isinf(lse)
    attn = torch.softmax(scores, dim=-1).masked_fill(dead.unsqueeze(-1), 0.0)
    if keep is not None:
        attn = attn.masked_fill(~keep, 0.0) / (1 - p)
    out = torch.einsum("bhqk,bhkd->bhqd", attn, vf)
    out.backward(do.float())
    return (out.detach(), lse.detach().masked_fill(dead, float("inf")), qf.grad, kf.grad, vf.grad,
            bf.grad if bias is not None else None)


@pytest.mark.parametrize("mask_type,Lq,Lk", [(0, 200, 328), (2, 200, 328), (1, 256, 256)])
def test_efficient_attention_pair_with_dropout(cuda_device, native_lib, mask_type, Lq, Lk):
    dev = cuda_device
    B, H, D, p = 2, 2, 128, 0.3
    q, k, v = rand((B, Lq, H, D), 1), rand((B, Lk, H, D), 2), rand((B, Lk, H, D), 3)
    do = torch.rand((B, Lq, H, D), generator=torch.Generator().manual_seed(4)).bfloat16()
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    out, lse, seed, off = ops._efficient_attention_forward(qd, kd, vd, None, None, None, None, p, mask_type, True)
    assert seed.numel() == 1 and off.numel() == 1
    dq, dk, dv, _ = ops._efficient_attention_backward(do.to(dev), qd, kd, vd, None, out.transpose(1, 2), None, None, Lk, Lq, lse,
                                                     p, seed, off, mask_type, False)
    assert ops.device_status() == 0
    keep = orc.dropout_keep_mask(int(seed), int(off), p, B, H, Lq, Lk)
    visible = None
    if mask_type == 1:
        visible = ~torch.ones(Lq, Lk, dtype=torch.bool).triu(1)
    elif mask_type == 2:
        visible = ~orc.causal_mask_bottom_right(Lq, Lk)
    t = lambda x: x.transpose(1, 2)
    o_r, l_r, dq_r, dk_r, dv_r, _ = fp32_attention(t(q), t(k), t(v), t(do), visible=visible, keep=keep, p=p)
    orc.assert_close_bf16(out, o_r, "out")
    orc.assert_close_lse(lse.view(H, B, Lq).permute(1, 0, 2), l_r)
    orc.assert_close_grad_bf16(t(dq), dq_r, "dq")
    orc.assert_close_grad_bf16(t(dk), dk_r, "dk")
    orc.assert_close_grad_bf16(t(dv), dv_r, "dv")


@pytest.mark.parametrize("with_dropout", [False, True])
def test_efficient_attention_with_cu_seqlens_and_bias(cuda_device, native_lib, with_dropout):
    """Packed sequences inside a [B, L] token grid together with a bias: sequence b reads bias[b, h, i, j] for its own
    query i and key j, and the bias gradient comes back in the same places (zero where no sequence reaches)."""
    dev = cuda_device
    B, L, H, D = 3, 256, 2, 128
    p = 0.25 if with_dropout else 0.0
    q, k, v, do = (rand((B, L, H, D), s) for s in (1, 2, 3, 4))
    bias = rand((B, H, L, L), 5)
    lens = [200, 256, 77]
    cu = [0, 200, 456, 533]
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    qd, kd, vd, bd = q.to(dev), k.to(dev), v.to(dev), bias.to(dev)
    out, lse, seed, off = ops._efficient_attention_forward(qd, kd, vd, bd, cu_t, cu_t, 256, p, 2, True)
    dq, dk, dv, db = ops._efficient_attention_backward(do.to(dev), qd, kd, vd, bd, out.transpose(1, 2), cu_t, cu_t, 256, 256, lse,
                                                      p, seed, off, 2, True)
    assert ops.device_status() == 0
    assert tuple(db.shape) == tuple(bias.shape)
    flat = lambda x: x.reshape(B * L, H, D)
    out_f = flat(out.transpose(1, 2))
    for b, n in enumerate(lens):
        sl = slice(cu[b], cu[b + 1])
        one = lambda x: flat(x)[sl].transpose(0, 1).unsqueeze(0)
        keep = orc.dropout_keep_mask(int(seed), int(off), p, B, H, n, n)[b:b + 1] if with_dropout else None
        vis = ~orc.causal_mask_bottom_right(n, n)
        o_r, l_r, dq_r, dk_r, dv_r, ds_r = fp32_attention(one(q), one(k), one(v), one(do), visible=vis,
                                                          bias=bias[b:b + 1, :, :n, :n], keep=keep, p=p)
        orc.assert_close_bf16(out_f[sl].transpose(0, 1).unsqueeze(0), o_r, f"out[{b}]")
        orc.assert_close_lse(lse[:, sl].unsqueeze(0), l_r, f"lse[{b}]")
        orc.assert_close_grad_bf16(flat(dq)[sl].transpose(0, 1).unsqueeze(0), dq_r, f"dq[{b}]")
        orc.assert_close_grad_bf16(flat(dk)[sl].transpose(0, 1).unsqueeze(0), dk_r, f"dk[{b}]")
        orc.assert_close_grad_bf16(flat(dv)[sl].transpose(0, 1).unsqueeze(0), dv_r, f"dv[{b}]")
        # the bias gradient is dS itself, element by element: P (dP - delta) with delta = rowsum(dO o O) taken from the
        # 16-bit O. In the first rows of a sequence P is close to 1 and the rounding of O (2^-9 per element, 128
        # elements) shows undiminished, so the absolute bound is 5e-2 here (dq, dk, dv average it out)
        orc.assert_close_grad_bf16(db[b:b + 1, :, :n, :n], ds_r, f"dbias[{b}]", max_abs=5e-2)
        assert float(db[b, :, n:, :].abs().max() if n < L else 0.0) == 0.0
        assert float(db[b, :, :, n:].abs().max() if n < L else 0.0) == 0.0


def test_flash_operator_pads_logsumexp_to_16_and_backward_cuts_it(cuda_device, native_lib):
    from torch_mlu_b200 import torch_glue
    torch_glue.load()
    dev = cuda_device
    B, H, Lq, Lk, D = 2, 2, 203, 203, 64
    q, k, v, do = rand((B, H, Lq, D), 1), rand((B, H, Lk, D), 2), rand((B, H, Lk, D), 3), rand((B, H, Lq, D), 4)
    o_ref, l_ref = orc.cpu_sdpa_forward(q, k, v, causal=True)
    want = orc.cpu_sdpa_backward(do, q, k, v, o_ref, l_ref, causal=True)
    for fwd, bwd in ((ops._scaled_dot_product_flash_attention, ops._scaled_dot_product_flash_attention_backward),
                     (torch.ops.b200_sdpa._scaled_dot_product_flash_attention,
                      torch.ops.b200_sdpa._scaled_dot_product_flash_attention_backward)):
        r = fwd(q.to(dev), k.to(dev), v.to(dev), 0.0, True, False)
        assert tuple(r[1].shape) == (B, H, 208)
        orc.assert_close_lse(r[1][..., :Lq], l_ref)
        assert float(r[1][..., Lq:].abs().max()) == 0.0
        orc.assert_close_bf16(r[0], o_ref, "out")
        grads = bwd(do.to(dev), q.to(dev), k.to(dev), v.to(dev), r[0], r[1], r[2], r[3], r[4], r[5], 0.0, True, r[6], r[7])
        for name, g, w in zip(("dq", "dk", "dv"), grads, want):
            orc.assert_close_grad_bf16(g, w, name)


def test_registered_packed_operator_returns_the_debug_mask(cuda_device, native_lib):
    from torch_mlu_b200 import torch_glue
    torch_glue.load()
    dev = cuda_device
    lens, Hq, Hkv, D, p = [100, 257, 31], 4, 2, 128, 0.3
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    q, k, v = rand((cu[-1], Hq, D), 1).to(dev), rand((cu[-1], Hkv, D), 2).to(dev), rand((cu[-1], Hkv, D), 3).to(dev)
    out, lse, seed, offset, debug = torch.ops.b200_sdpa._flash_attention_forward(q, k, v, cu_t, cu_t, max(lens), max(lens), p,
                                                                                False, True)
    assert tuple(debug.shape) == (len(lens), Hq, max(lens), max(lens)) and debug.dtype == q.dtype
    for b, n in enumerate(lens):
        want = orc.dropout_keep_mask(int(seed), int(offset), p, len(lens), Hq, n, n)[b]
        assert torch.equal((debug[b, :, :n, :n] > 0).cpu(), want), f"sequence {b}"
        assert float(debug[b, :, n:, :].abs().max() if n < max(lens) else 0.0) == 0.0
    assert torch.ops.b200_sdpa._device_status(-1) == 0


def test_backward_takes_the_masks_its_forward_left(cuda_device, native_lib):
    """Same gradients, bit for bit, whether the backward finds the forward's keep-masks or draws them again; and a
    hit launches one kernel less (the keep-mask kernel)."""
    dev = cuda_device
    B, H, L, D, p = 2, 2, 384, 128, 0.2
    q, k, v, do = (rand((B, H, L, D), s).to(dev) for s in (1, 2, 3, 4))
    r = ops._scaled_dot_product_flash_attention(q, k, v, p, True, False)
    n0 = _cabi.launch_count()
    hit = ops._scaled_dot_product_flash_attention_backward(do, q, k, v, r[0], r[1], r[2], r[3], r[4], r[5], p, True, r[6], r[7])
    n1 = _cabi.launch_count()
    miss = ops._scaled_dot_product_flash_attention_backward(do, q, k, v, r[0], r[1], r[2], r[3], r[4], r[5], p, True, r[6], r[7])
    n2 = _cabi.launch_count()
    assert (n2 - n1) - (n1 - n0) == 1
    assert torch.equal(hit[1], miss[1]) and torch.equal(hit[2], miss[2])
    orc.assert_close_grad_bf16(hit[0], miss[0].float(), "dq from kept masks vs redrawn masks")
    assert dropout._LastForward.take(dev, ("nothing",)) is None


def test_a_wait_that_runs_out_reports_device_timeout_and_the_context_survives(cuda_device, native_lib):
    """The self-test kernel waits 50 us on a barrier nobody arrives on - nothing is in flight - gives up the way the
    attention kernels do, and returns. The status word says DEVICE_TIMEOUT until it is read; the next call is clean."""
    dev = cuda_device
    lib = native_lib
    assert ops.device_status(dev) == 0
    word = ops._Workspace.status_word(dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    _cabi.check(lib.sdpa_b200_selftest_wait_timeout(word.data_ptr(), 50, stream), "selftest")
    # a healthy attention call in between neither hides nor clears the report
    q = rand((1, 2, 256, 128), 1).to(dev)
    out, lse = ops.gqa_prefill(q, q, q, is_causal=True)
    with pytest.raises(_cabi.SdpaError, match="DEVICE_TIMEOUT"):
        ops.check_device_status(dev)
    assert ops.device_status(dev) == 0
    out2, lse2 = ops.gqa_prefill(q, q, q, is_causal=True)
    assert ops.device_status(dev) == 0
    assert torch.equal(out, out2) and torch.equal(lse, lse2)
    o_ref, l_ref = orc.cpu_sdpa_forward(q.cpu(), q.cpu(), q.cpu(), causal=True)
    orc.assert_close_bf16(out2, o_ref, "out after a reported time-out")
    # through a workspace's own first word as well (the default when no status word is given)
    ws = torch.zeros(256, dtype=torch.uint8, device=dev)
    _cabi.check(lib.sdpa_b200_selftest_wait_timeout(ws.data_ptr(), 50, stream), "selftest")
    st = ctypes.c_int(0)
    _cabi.check(lib.sdpa_b200_read_device_status(ws.data_ptr(), stream, ctypes.byref(st)), "read")
    assert st.value == _cabi.DEVICE_TIMEOUT
    # argument checks
    assert lib.sdpa_b200_selftest_wait_timeout(None, 50, stream) == _cabi.INVALID_ARG
    assert lib.sdpa_b200_selftest_wait_timeout(word.data_ptr(), 0, stream) == _cabi.INVALID_ARG


def test_status_word_through_the_registered_operators(cuda_device, native_lib):
    from torch_mlu_b200 import torch_glue
    torch_glue.load()
    assert torch.ops.b200_sdpa._device_status(0) == 0


@pytest.mark.parametrize("margin", [8, 32, 1000])
def test_sm_margin_leaves_the_result_alone(cuda_device, native_lib, margin):
    """`sm_margin` only shrinks the persistent forward grid (what is left over serves a collective on another
    stream); the units are handed out by a counter, so any grid size - down to one CTA - gives the same bits."""
    q, k, v = rand((2, 4, 640, 128), 31), rand((2, 4, 640, 128), 32), rand((2, 4, 640, 128), 33)
    qd, kd, vd = (t.to(cuda_device) for t in (q, k, v))
    out0, lse0 = ops.gqa_prefill(qd, kd, vd, is_causal=True)
    out1, lse1 = ops.gqa_prefill(qd, kd, vd, is_causal=True, sm_margin=margin)
    assert torch.equal(out0, out1) and torch.equal(lse0, lse1)
    o_ref, l_ref = orc.cpu_sdpa_forward(q, k, v, causal=True)
    orc.assert_close_bf16(out1, o_ref, "out")
    orc.assert_close_lse(lse1, l_ref)
