"""The dispatcher glue on a GPU: the b200_sdpa operators (reference schemas) with autograd, and
the opt-in aten overrides that put F.scaled_dot_product_attention on these kernels."""
import pytest
import torch
import torch.nn.functional as F

from oracle import sdpa_oracle as orc
from torch_mlu_b200 import _cabi, backends, torch_glue

pytestmark = pytest.mark.gpu


def rand(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g).bfloat16()


def test_registered_ops_forward_backward_autograd(cuda_device, native_lib):
    torch_glue.load()
    dev = cuda_device
    q, k, v, do = (rand((2, 4, 384, 128), s) for s in (1, 2, 3, 4))
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    res = torch.ops.b200_sdpa._scaled_dot_product_flash_attention(qd, kd, vd, 0.0, True, False)
    out, lse = res[0], res[1]
    assert len(res) == 9 and res[4] == 384 and res[5] == 384
    out.backward(do.to(dev))
    o_ref, l_ref = orc.cpu_sdpa_forward(q, k, v, causal=True)
    dq, dk, dv = orc.cpu_sdpa_backward(do, q, k, v, o_ref, l_ref, causal=True)
    orc.assert_close_bf16(out, o_ref, "out")
    orc.assert_close_lse(lse, l_ref)
    orc.assert_close_grad_bf16(qd.grad, dq, "dq")
    orc.assert_close_grad_bf16(kd.grad, dk, "dk")
    orc.assert_close_grad_bf16(vd.grad, dv, "dv")


def test_registered_varlen_op_autograd(cuda_device, native_lib):
    torch_glue.load()
    dev = cuda_device
    lens = [100, 260, 33]
    cu = [0, 100, 360, 393]
    q, k, v, do = rand((393, 4, 128), 1), rand((393, 2, 128), 2), rand((393, 2, 128), 3), rand((393, 4, 128), 4)
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    out, lse, *_ = torch.ops.b200_sdpa._flash_attention_forward(qd, kd, vd, cu_t, cu_t, max(lens), max(lens), 0.0, True, False)
    out.backward(do.to(dev))
    o_ref, l_ref = orc.varlen_forward(q, k, v, cu, cu, causal=True)
    dq, dk, dv = orc.varlen_backward(do, q, k, v, cu, cu, causal=True)
    orc.assert_close_bf16(out, o_ref, "out")
    orc.assert_close_lse(lse, l_ref)
    orc.assert_close_grad_bf16(qd.grad, dq, "dq")
    orc.assert_close_grad_bf16(kd.grad, dk, "dk")
    orc.assert_close_grad_bf16(vd.grad, dv, "dv")


def test_functional_sdpa_reaches_these_kernels_when_overridden(cuda_device, native_lib):
    """Same call pattern as the reference tests: F.scaled_dot_product_attention inside
    sdp_kernel(enable_flash=True, enable_math=False, enable_mem_efficient=False)
    (test/torch_ops/test_scaled_dot_product_attention.py:630-640)."""
    dev = cuda_device
    q, k, v, do = (rand((1, 16, 512, 128), s) for s in (1, 2, 3, 4))
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    torch_glue.install_aten_overrides()
    try:
        before = _cabi.launch_count()
        with backends.sdp_kernel(enable_flash=True, enable_math=False, enable_mem_efficient=False):
            out = F.scaled_dot_product_attention(qd, kd, vd, is_causal=True)
        out.backward(do.to(dev))
        torch.cuda.synchronize()
        assert _cabi.launch_count() - before == 4  # forward + (preprocess, dK/dV, dQ)
    finally:
        torch_glue.remove_aten_overrides()
    o_ref, l_ref = orc.cpu_sdpa_forward(q, k, v, causal=True)
    dq, dk, dv = orc.cpu_sdpa_backward(do, q, k, v, o_ref, l_ref, causal=True)
    orc.assert_close_bf16(out, o_ref, "out")
    orc.assert_close_grad_bf16(qd.grad, dq, "dq")
    orc.assert_close_grad_bf16(kd.grad, dk, "dk")
    orc.assert_close_grad_bf16(vd.grad, dv, "dv")
    # with the overrides removed the stock kernel is back (no launches of this library)
    before = _cabi.launch_count()
    with backends.sdp_kernel(enable_flash=True, enable_math=False, enable_mem_efficient=False):
        F.scaled_dot_product_attention(qd.detach(), kd.detach(), vd.detach(), is_causal=True)
    torch.cuda.synchronize()
    assert _cabi.launch_count() == before


def test_glue_rejects_what_the_reference_rejects(cuda_device, native_lib):
    torch_glue.load()
    dev = cuda_device
    q = rand((1, 2, 64, 128), 1).to(dev)
    with pytest.raises(RuntimeError, match="same number of heads"):
        torch.ops.b200_sdpa._scaled_dot_product_flash_attention(q, q[:, :1], q[:, :1])
    with pytest.raises(RuntimeError, match="fp16 and bf16"):
        torch.ops.b200_sdpa._scaled_dot_product_flash_attention(q.float(), q.float(), q.float())
    with pytest.raises(RuntimeError, match="dropout_p must be inside"):
        torch.ops.b200_sdpa._scaled_dot_product_flash_attention(q, q, q, 1.0)
    wide = torch.cat([q, q, q[..., :64]], dim=-1)  # head_dim 320: beyond what the reference admits (sdp_utils.h:231-255)
    with pytest.raises(RuntimeError, match="at most 256"):
        torch.ops.b200_sdpa._scaled_dot_product_flash_attention(wide, wide, wide)


@pytest.mark.parametrize("amp_dtype", [torch.bfloat16, torch.float16])
def test_autocast_casts_fp32_inputs_like_the_reference(cuda_device, native_lib, amp_dtype):
    """aten/autocast_mode.cpp:147 puts _scaled_dot_product_flash_attention on the
    lower_precision_fp list: fp32 inputs run in the autocast dtype, gradients come back in fp32."""
    torch_glue.load()
    dev = cuda_device
    g = torch.Generator().manual_seed(11)
    q, k, v, do = (torch.randn((1, 2, 256, 128), generator=g) for _ in range(4))
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    with torch.autocast("cuda", dtype=amp_dtype):
        out = torch.ops.b200_sdpa._scaled_dot_product_flash_attention(qd, kd, vd, 0.0, True, False)[0]
    assert out.dtype == amp_dtype
    out.backward(do.to(dev).to(amp_dtype))
    assert qd.grad.dtype == torch.float32
    ql, kl, vl, dl = (t.to(amp_dtype) for t in (q, k, v, do))
    o_ref, l_ref = orc.cpu_sdpa_forward(ql, kl, vl, causal=True)
    dq, dk, dv = orc.cpu_sdpa_backward(dl, ql, kl, vl, o_ref, l_ref, causal=True)
    orc.assert_close_bf16(out, o_ref, "out")
    orc.assert_close_grad_bf16(qd.grad, dq, "dq")
    orc.assert_close_grad_bf16(kd.grad, dk, "dk")
    orc.assert_close_grad_bf16(vd.grad, dv, "dv")


def _attention_with_mask(q, k, v, keep, p, causal, dtype=torch.float32):
    qf, kf, vf = (t.to(dtype).detach().requires_grad_(True) for t in (q, k, v))
    scores = torch.einsum("bhtd,bhsd->bhts", qf * (q.shape[-1] ** -0.5), kf)
    if causal:
        scores = scores.masked_fill(orc.causal_mask_bottom_right(q.shape[2], k.shape[2]), float("-inf"))
    attn = torch.softmax(scores, dim=-1).masked_fill(~keep, 0.0) / (1.0 - p)
    return torch.einsum("bhts,bhsd->bhtd", attn, vf), (qf, kf, vf)


def test_dropout_through_the_registered_operator_and_autograd(cuda_device, native_lib):
    """dropout_p > 0 with return_debug_mask, as the reference tests call it (test_...py:1018-1026): the operator
    returns the pattern and the Philox pair; autograd's backward replays the pattern from the pair."""
    torch_glue.load()
    dev = cuda_device
    p = 0.22
    q, k, v = (rand((2, 3, 260, 128), s) for s in (1, 2, 3))
    do = torch.rand((2, 3, 260, 128), generator=torch.Generator().manual_seed(4)).bfloat16()
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    res = torch.ops.b200_sdpa._scaled_dot_product_flash_attention(qd, kd, vd, p, True, True)
    out, seed, offset, debug = res[0], res[6], res[7], res[8]
    assert seed.numel() == 1 and offset.numel() == 1 and tuple(debug.shape) == (2, 3, 260, 260)
    keep = (debug > 0).cpu()
    visible = ~orc.causal_mask_bottom_right(260, 260)
    assert torch.equal(keep & visible, orc.dropout_keep_mask(int(seed), int(offset), p, 2, 3, 260, 260) & visible)
    out.backward(do.to(dev))
    ref, (qf, kf, vf) = _attention_with_mask(q, k, v, keep, p, True)
    ref.backward(do.float())
    lp, (ql, kl, vl) = _attention_with_mask(q, k, v, keep, p, True, torch.bfloat16)
    lp.backward(do)
    orc.assert_close_bf16(out, ref.detach(), "out")
    orc.assert_close_reference_rule(qd.grad, qf.grad, ql.grad, "dq", fudge=4)
    orc.assert_close_reference_rule(kd.grad, kf.grad, kl.grad, "dk")
    orc.assert_close_reference_rule(vd.grad, vf.grad, vl.grad, "dv")


def test_functional_sdpa_with_dropout_uses_the_cuda_generator(cuda_device, native_lib):
    """F.scaled_dot_product_attention(dropout_p=...) on the overridden aten operators: the pattern comes from the
    device generator's (seed, offset), which the test reads before the call to rebuild the expected result."""
    dev = cuda_device
    p = 0.3
    q, k, v = (rand((1, 4, 256, 128), s) for s in (1, 2, 3))
    do = torch.rand((1, 4, 256, 128), generator=torch.Generator().manual_seed(4)).bfloat16()
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    torch_glue.install_aten_overrides()
    try:
        torch.cuda.manual_seed(4242)
        gen = torch.cuda.default_generators[dev.index or 0]
        seed, offset = gen.initial_seed(), gen.get_offset()
        with backends.sdp_kernel(enable_flash=True, enable_math=False, enable_mem_efficient=False):
            out = F.scaled_dot_product_attention(qd, kd, vd, dropout_p=p, is_causal=True)
            again = F.scaled_dot_product_attention(qd, kd, vd, dropout_p=p, is_causal=True)
        out.backward(do.to(dev))
    finally:
        torch_glue.remove_aten_overrides()
    assert not torch.equal(out, again)          # the generator moved on
    keep = orc.dropout_keep_mask(seed, offset, p, 1, 4, 256, 256)
    ref, (qf, kf, vf) = _attention_with_mask(q, k, v, keep, p, True)
    ref.backward(do.float())
    orc.assert_close_bf16(out, ref.detach(), "out")
    orc.assert_close_grad_bf16(qd.grad, qf.grad, "dq")
    orc.assert_close_grad_bf16(kd.grad, kf.grad, "dk")
    orc.assert_close_grad_bf16(vd.grad, vf.grad, "dv")


def test_packed_operator_with_dropout_and_autograd(cuda_device, native_lib):
    """b200_sdpa::_flash_attention_forward with dropout_p > 0: the Philox pair comes back, autograd's backward
    replays the pattern, and everything matches fp32 math with the pattern rebuilt on the CPU."""
    torch_glue.load()
    dev = cuda_device
    p, H, D = 0.22, 2, 128
    lens = [130, 257]
    cu = [0, 130, 387]
    q, k, v = (rand((387, H, D), s) for s in (1, 2, 3))
    do = torch.rand((387, H, D), generator=torch.Generator().manual_seed(4)).bfloat16()
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    out, lse, seed, offset, _ = torch.ops.b200_sdpa._flash_attention_forward(qd, kd, vd, cu_t, cu_t, 257, 257, p, True, False)
    assert seed.numel() == 1 and offset.numel() == 1
    out.backward(do.to(dev))
    for b, L in enumerate(lens):
        sl = slice(cu[b], cu[b + 1])
        one = lambda x: x[sl].transpose(0, 1).unsqueeze(0)
        keep = orc.dropout_keep_mask(int(seed), int(offset), p, len(lens), H, L, L)[b:b + 1]
        ref, (qf, kf, vf) = _attention_with_mask(one(q), one(k), one(v), keep, p, True)
        ref.backward(one(do).float())
        orc.assert_close_bf16(one(out), ref.detach(), f"out[{b}]")
        orc.assert_close_grad_bf16(one(qd.grad), qf.grad, f"dq[{b}]")
        orc.assert_close_grad_bf16(one(kd.grad), kf.grad, f"dk[{b}]")
        orc.assert_close_grad_bf16(one(vd.grad), vf.grad, f"dv[{b}]")
