"""GPU parity of every kernel for IEEE half inputs (the reference accepts fp16 and bf16:
torch_mlu/csrc/aten/operators/cnnl/internal/FlashAttention_internal.cpp:74-80), against the CPU
oracle on the same fp16-rounded inputs, through the C ABI.

Tolerances are those of the bf16 tests (out / grads max-abs 2e-2, mean-abs 2e-3; lse 1e-5);
fp16 has three more mantissa bits, so they hold with margin.
"""
import pytest
import torch

from oracle import sdpa_oracle as orc
from torch_mlu_b200 import ops, ring

pytestmark = pytest.mark.gpu


def rand(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g).half()


@pytest.mark.parametrize("B,Hq,Hkv,Lq,Lk,D,causal", [
    (2, 4, 4, 512, 512, 128, True),
    (1, 8, 2, 300, 700, 128, True),
    (1, 2, 2, 257, 255, 128, False),
    (1, 2, 2, 1024, 512, 64, False),
    (2, 8, 2, 384, 384, 64, True),
    (1, 1, 1, 1, 1, 128, True),
])
def test_f16_forward_backward(cuda_device, native_lib, B, Hq, Hkv, Lq, Lk, D, causal):
    dev = cuda_device
    q, k, v, dout = rand((B, Hq, Lq, D), 1), rand((B, Hkv, Lk, D), 2), rand((B, Hkv, Lk, D), 3), rand((B, Hq, Lq, D), 4)
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    out, lse = ops.gqa_prefill(qd, kd, vd, is_causal=causal)
    assert out.dtype == torch.float16
    dq, dk, dv = ops._dense_backward(dout.to(dev), qd, kd, vd, out, lse, causal, ops.calculate_scale(qd, None))
    assert ops.device_status() == 0
    o_ref, l_ref = orc.cpu_sdpa_forward(q, k, v, causal=causal)
    orc.assert_close_bf16(out, o_ref, "out")
    orc.assert_close_lse(lse, l_ref)
    want = orc.cpu_sdpa_backward(dout, q, k, v, o_ref, l_ref, causal=causal)
    for name, g, w in zip(("dq", "dk", "dv"), (dq, dk, dv), want):
        assert g.dtype == torch.float16
        orc.assert_close_grad_bf16(g, w, name)


def test_f16_large_scores_stay_finite(cuda_device, native_lib):
    """Unnormalised probabilities reach 2^8 before a lazy rescale; that and a large-magnitude V
    must stay inside the fp16 range."""
    dev = cuda_device
    q, k = rand((1, 2, 512, 128), 1) * 3, rand((1, 2, 512, 128), 2) * 3
    v = rand((1, 2, 512, 128), 3) * 100
    out, lse = ops.gqa_prefill(q.to(dev), k.to(dev), v.to(dev), is_causal=True)
    assert torch.isfinite(out.float()).all()
    o_ref, l_ref = orc.cpu_sdpa_forward(q, k, v, causal=True)
    rel = (out.float().cpu() - o_ref).abs().max() / o_ref.abs().max()
    assert rel < 2e-3, rel
    orc.assert_close_lse(lse, l_ref, max_abs=2e-4)


def test_f16_varlen(cuda_device, native_lib):
    dev = cuda_device
    lens, Hq, Hkv = [100, 300, 257, 128], 4, 2
    total = sum(lens)
    q, k, v, dout = rand((total, Hq, 128), 1), rand((total, Hkv, 128), 2), rand((total, Hkv, 128), 3), rand((total, Hq, 128), 4)
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    out, lse, seed, off, _ = ops._flash_attention_forward(qd, kd, vd, cu_t, cu_t, max(lens), max(lens), 0.0, True, False)
    dq, dk, dv = ops._flash_attention_backward(dout.to(dev), qd, kd, vd, out, lse, cu_t, cu_t, max(lens), max(lens), 0.0,
                                               True, seed, off)
    assert ops.device_status() == 0
    o_ref, l_ref = orc.varlen_forward(q, k, v, cu, cu, causal=True)
    orc.assert_close_bf16(out, o_ref, "out")
    for name, g, w in zip(("dq", "dk", "dv"), (dq, dk, dv), orc.varlen_backward(dout, q, k, v, cu, cu, causal=True)):
        orc.assert_close_grad_bf16(g, w, name)


@pytest.mark.parametrize("B,Hq,Hkv,Lk,D,splits", [
    (2, 8, 2, 1000, 128, 4), (2, 32, 2, 777, 128, 3), (1, 4, 4, 4096, 64, 0), (3, 8, 8, 1, 128, 1),
])
def test_f16_decode(cuda_device, native_lib, B, Hq, Hkv, Lk, D, splits):
    dev = cuda_device
    q, k, v = rand((B, Hq, 1, D), 1), rand((B, Hkv, Lk, D), 2), rand((B, Hkv, Lk, D), 3)
    out, lse = ops.decode_attention(q.to(dev), k.to(dev), v.to(dev), num_splits=splits)
    assert out.dtype == torch.float16
    o_ref, l_ref = orc.cpu_sdpa_forward(q, k, v, causal=False)
    orc.assert_close_bf16(out, o_ref, "out")
    orc.assert_close_lse(lse, l_ref)


def test_f16_merge_partial(cuda_device, native_lib):
    dev = cuda_device
    g = torch.Generator().manual_seed(5)
    B, H, L, D = 2, 3, 200, 128
    o_acc = torch.randn(B, H, L, D, generator=g).to(dev)
    lse_acc = torch.randn(B, H, L, generator=g).to(dev)
    o_part = torch.randn(B, H, L, D, generator=g).half().to(dev)
    lse_part = torch.randn(B, H, L, generator=g).to(dev)
    want_o, want_l = o_acc.clone(), lse_acc.clone()
    ring.merge_partial_reference(want_o, want_l, o_part, lse_part)
    ring.merge_partial(o_acc, lse_acc, o_part, lse_part)
    assert torch.allclose(o_acc, want_o, atol=1e-5) and torch.allclose(lse_acc, want_l, atol=1e-5)


def test_mixed_dtypes_are_refused(cuda_device, native_lib):
    dev = cuda_device
    q = rand((1, 2, 128, 128), 1).to(dev)
    with pytest.raises(RuntimeError, match="same dtype"):
        ops.gqa_prefill(q, q.bfloat16(), q.bfloat16(), is_causal=False)
