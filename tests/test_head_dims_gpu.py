"""GPU parity for head dims between the two the kernels are built for (64 and 128 columns).

The reference accepts any head_dim that is a multiple of 8 (sdp_utils.h:231-255). Here such a head
dim runs in the next larger kernel: TMA loads pad the rows with zeros, TMA stores clip them, and the
two paths that write rows without TMA (rows without a visible key, ragged varlen tiles) stop at the
real row length.
"""
import pytest
import torch

from oracle import sdpa_oracle as orc
from torch_mlu_b200 import ops

pytestmark = pytest.mark.gpu


def rand(shape, seed, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g).to(dtype)


@pytest.mark.parametrize("D", [8, 40, 72, 96, 120])
@pytest.mark.parametrize("Lq,Lk,causal", [(300, 300, True), (130, 257, False), (200, 70, True)])
def test_forward_backward_dense(cuda_device, native_lib, D, Lq, Lk, causal):
    dev = cuda_device
    B, Hq, Hkv = 2, 4, 2
    q, k, v, dout = rand((B, Hq, Lq, D), 1), rand((B, Hkv, Lk, D), 2), rand((B, Hkv, Lk, D), 3), rand((B, Hq, Lq, D), 4)
    qd, kd, vd, dd = q.to(dev), k.to(dev), v.to(dev), dout.to(dev)
    out, lse = ops.gqa_prefill(qd, kd, vd, is_causal=causal)
    dq, dk, dv = ops._dense_backward(dd, qd, kd, vd, out, lse, causal, ops.calculate_scale(qd, None))
    assert ops.device_status() == 0
    if causal and Lq != Lk:
        o_ref, l_ref = orc.attention_math(q, k, v, causal=True)  # bottom-right aligned, like the kernels
        want = orc.attention_math_backward(q, k, v, dout, causal=True)
    else:
        o_ref, l_ref = orc.cpu_sdpa_forward(q, k, v, causal=causal)
        want = orc.cpu_sdpa_backward(dout, q, k, v, o_ref, l_ref, causal=causal)
    orc.assert_close_bf16(out, o_ref, "out")
    orc.assert_close_lse(lse, l_ref)
    for name, g, w in zip(("dq", "dk", "dv"), (dq, dk, dv), want):
        orc.assert_close_grad_bf16(g, w, name)


@pytest.mark.parametrize("D", [72, 104])
def test_varlen_ragged_tiles(cuda_device, native_lib, D):
    # ragged tiles are written row by row from registers: a store past column D would land in the next head's row
    dev = cuda_device
    lens, Hq, Hkv = [100, 300, 257, 1], 4, 2
    total = sum(lens)
    q, k, v, dout = rand((total, Hq, D), 1), rand((total, Hkv, D), 2), rand((total, Hkv, D), 3), rand((total, Hq, D), 4)
    cu = [0]
    for l in lens:
        cu.append(cu[-1] + l)
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    out, lse, seed, off, _ = ops._flash_attention_forward(qd, kd, vd, cu_t, cu_t, max(lens), max(lens), 0.0, True, False)
    dq, dk, dv = ops._flash_attention_backward(dout.to(dev), qd, kd, vd, out, lse, cu_t, cu_t, max(lens), max(lens), 0.0,
                                               True, seed, off)
    assert ops.device_status() == 0
    o_ref, l_ref = orc.varlen_forward(q, k, v, cu, cu, causal=True)
    orc.assert_close_bf16(out, o_ref, "out")
    orc.assert_close_lse(lse, l_ref)
    for name, g, w in zip(("dq", "dk", "dv"), (dq, dk, dv), orc.varlen_backward(dout, q, k, v, cu, cu, causal=True)):
        orc.assert_close_grad_bf16(g, w, name)


def test_decode_shape_with_other_head_dim_takes_the_tile_kernel(cuda_device, native_lib):
    dev = cuda_device
    B, H, Lk, D = 3, 4, 1000, 96
    q, k, v = rand((B, H, 1, D), 1), rand((B, H, Lk, D), 2), rand((B, H, Lk, D), 3)
    # one query row: head_dim 64 or 128 would pick the streaming decode kernel here
    out, lse, *_ = ops._scaled_dot_product_flash_attention(q.to(dev), k.to(dev), v.to(dev))
    assert ops.device_status() == 0
    lse = lse[..., :1]
    o_ref, l_ref = orc.cpu_sdpa_forward(q, k, v, causal=False)
    orc.assert_close_bf16(out, o_ref, "out")
    orc.assert_close_lse(lse, l_ref)


def test_fp16_head_dim_80(cuda_device, native_lib):
    dev = cuda_device
    q, k, v = (rand((1, 2, 260, 80), s, torch.float16) for s in (1, 2, 3))
    out, lse = ops.gqa_prefill(q.to(dev), k.to(dev), v.to(dev), is_causal=True)
    assert ops.device_status() == 0
    o_ref, l_ref = orc.cpu_sdpa_forward(q, k, v, causal=True)
    orc.assert_close_bf16(out, o_ref, "out")
    orc.assert_close_lse(lse, l_ref)
