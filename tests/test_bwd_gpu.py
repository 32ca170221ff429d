"""GPU parity of the backward kernels (dQ, dK, dV) against the CPU oracle, through the C ABI.

Tolerances for bf16 gradients vs the fp32 oracle on the same bf16-rounded inputs: mean-abs
2e-3 and max-abs 2e-2, the latter widened to 1e-2*|want| only where |want| > 2 (bf16 cannot
represent such values to 2e-2; see oracle.sdpa_oracle.assert_close_grad_bf16).
"""
import os

import pytest
import torch

from oracle import sdpa_oracle as orc
from test_oracle import GOLDEN, load_golden
from torch_mlu_b200 import ops, workloads

pytestmark = pytest.mark.gpu


def rand(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g).bfloat16()


def run_fwd_bwd(dev, q, k, v, dout, causal, scale=None, deterministic=None):
    qd, kd, vd, dd = q.to(dev), k.to(dev), v.to(dev), dout.to(dev)
    out, lse = ops.gqa_prefill(qd, kd, vd, is_causal=causal, scale=scale)
    dq, dk, dv = ops._dense_backward(dd, qd, kd, vd, out, lse, causal, ops.calculate_scale(qd, scale),
                                     deterministic=deterministic)
    assert ops.device_status() == 0
    return out, lse, dq, dk, dv


def check_grads(got, want, names=("dq", "dk", "dv")):
    for name, g, w in zip(names, got, want):
        assert g.shape == w.shape, name
        orc.assert_close_grad_bf16(g, w, name)


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: os.path.basename(p)[14:-4])
def test_backward_matches_reference_golden(cuda_device, native_lib, path):
    g = load_golden(path)
    out, lse, dq, dk, dv = run_fwd_bwd(cuda_device, g["q"], g["k"], g["v"], g["dout"], g["causal"], g["scale"])
    check_grads((dq, dk, dv), (g["dq"], g["dk"], g["dv"]))


@pytest.mark.parametrize("B,Hq,Hkv,Lq,Lk,causal", [
    (1, 1, 1, 128, 128, False),
    (2, 4, 4, 512, 512, True),
    (1, 2, 2, 1024, 512, False),
    (1, 2, 2, 1000, 1000, True),
    (1, 2, 2, 300, 700, True),
    (1, 2, 2, 700, 300, True),     # leading query rows see no key: their dq must be 0
    (1, 2, 2, 17, 129, False),
    (1, 1, 1, 1, 1, True),
    (2, 8, 2, 384, 384, True),     # GQA: dk/dv summed over 4 query heads
    (1, 8, 1, 256, 512, False),    # MQA
    (1, 2, 2, 257, 255, True),
])
def test_backward_dense_shapes(cuda_device, native_lib, B, Hq, Hkv, Lq, Lk, causal):
    q, k, v = rand((B, Hq, Lq, 128), 1), rand((B, Hkv, Lk, 128), 2), rand((B, Hkv, Lk, 128), 3)
    dout = rand((B, Hq, Lq, 128), 4)
    out, lse, dq, dk, dv = run_fwd_bwd(cuda_device, q, k, v, dout, causal)
    o_ref, l_ref = orc.cpu_sdpa_forward(q, k, v, causal=causal)
    want = orc.cpu_sdpa_backward(dout, q, k, v, o_ref, l_ref, causal=causal)
    check_grads((dq, dk, dv), want)


@pytest.mark.parametrize("B,Hq,Hkv,Lq,Lk,causal", [
    (2, 4, 4, 512, 512, True),
    (1, 8, 2, 300, 700, True),
    (1, 2, 2, 257, 255, False),
])
def test_backward_head_dim_64(cuda_device, native_lib, B, Hq, Hkv, Lq, Lk, causal):
    g = torch.Generator().manual_seed(6)
    q = torch.randn((B, Hq, Lq, 64), generator=g).bfloat16()
    k = torch.randn((B, Hkv, Lk, 64), generator=g).bfloat16()
    v = torch.randn((B, Hkv, Lk, 64), generator=g).bfloat16()
    dout = torch.randn((B, Hq, Lq, 64), generator=g).bfloat16()
    out, lse, dq, dk, dv = run_fwd_bwd(cuda_device, q, k, v, dout, causal)
    o_ref, l_ref = orc.cpu_sdpa_forward(q, k, v, causal=causal)
    check_grads((dq, dk, dv), orc.cpu_sdpa_backward(dout, q, k, v, o_ref, l_ref, causal=causal))


def test_backward_reference_operator_surface_and_scale(cuda_device, native_lib):
    """_scaled_dot_product_flash_attention_backward takes the forward's 9-tuple pieces
    (attention.cpp:205-297); scale = 1/D as in the reference sweep."""
    dev = cuda_device
    q, k, v, dout = (rand((2, 4, 512, 128), s) for s in (1, 2, 3, 4))
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    scale = 1.0 / 128
    out, lse, cq, ck, mq, mk, seed, off, _ = ops._scaled_dot_product_flash_attention(qd, kd, vd, 0.0, True, False, scale=scale)
    # a non-contiguous grad_out view is accepted
    dd = dout.to(dev).transpose(1, 2).contiguous().transpose(1, 2)
    dq, dk, dv = ops._scaled_dot_product_flash_attention_backward(dd, qd, kd, vd, out, lse, cq, ck, mq, mk, 0.0, True,
                                                                  seed, off, scale=scale)
    assert dq.shape == q.shape and dk.shape == k.shape and dv.shape == v.shape
    o_ref, l_ref = orc.cpu_sdpa_forward(q, k, v, causal=True, scale=scale)
    check_grads((dq, dk, dv), orc.cpu_sdpa_backward(dout, q, k, v, o_ref, l_ref, causal=True, scale=scale))


@pytest.mark.parametrize("lens,Hq,Hkv,causal", [
    ([100, 300, 257, 128], 4, 2, True),
    ([512, 64, 1000], 4, 1, False),
    ([1, 2, 3, 255, 256, 257], 2, 2, True),
])
def test_backward_varlen(cuda_device, native_lib, lens, Hq, Hkv, causal):
    dev = cuda_device
    total = sum(lens)
    q, k, v, dout = rand((total, Hq, 128), 1), rand((total, Hkv, 128), 2), rand((total, Hkv, 128), 3), rand((total, Hq, 128), 4)
    cu = [0]
    for l in lens:
        cu.append(cu[-1] + l)
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    out, lse, seed, off, _ = ops._flash_attention_forward(qd, kd, vd, cu_t, cu_t, max(lens), max(lens), 0.0, causal, False)
    dq, dk, dv = ops._flash_attention_backward(dout.to(dev), qd, kd, vd, out, lse, cu_t, cu_t, max(lens), max(lens), 0.0,
                                               causal, seed, off)
    assert ops.device_status() == 0
    check_grads((dq, dk, dv), orc.varlen_backward(dout, q, k, v, cu, cu, causal=causal))


def test_backward_is_deterministic(cuda_device, native_lib):
    """With `deterministic` every gradient comes back with the same bits on every call (the dK/dV and dQ kernels sum
    in a fixed order). The fused kernel keeps that promise for dK and dV; its dQ sums are formed by floating-point
    reductions in global memory and repeat only to fp32 rounding."""
    q, k, v, dout = (rand((1, 4, 640, 128), s) for s in (1, 2, 3, 4))
    a = run_fwd_bwd(cuda_device, q, k[:, :2], v[:, :2], dout, True, deterministic=True)
    b = run_fwd_bwd(cuda_device, q, k[:, :2], v[:, :2], dout, True, deterministic=True)
    for x, y in zip(a, b):
        assert torch.equal(x, y)
    c = run_fwd_bwd(cuda_device, q, k[:, :2], v[:, :2], dout, True, deterministic=False)
    d = run_fwd_bwd(cuda_device, q, k[:, :2], v[:, :2], dout, True, deterministic=False)
    assert torch.equal(c[3], d[3]) and torch.equal(c[4], d[4])
    assert orc.error_stats(c[2], d[2])[0] <= 2e-2 and orc.error_stats(c[2], a[2])[0] <= 2e-2
    # torch's global switch selects the same path
    torch.use_deterministic_algorithms(True)
    try:
        e = run_fwd_bwd(cuda_device, q, k[:, :2], v[:, :2], dout, True)
    finally:
        torch.use_deterministic_algorithms(False)
    for x, y in zip(a, e):
        assert torch.equal(x, y)


def test_config3_sampled_heads_and_linearity(cuda_device, native_lib):
    """BASELINE config 3 at full size (B8 H16 L2048 D128 causal, seed 2): oracle parity on
    sampled (batch, head) pairs, and a size-independent property on everything: the backward
    is linear in dO, so grads(2*dO) == 2*grads(dO) bit for bit (scaling by 2 is exact in bf16)."""
    dev = cuda_device
    c = workloads.config3_causal_fwd_bwd()
    qd, kd, vd, dd = c.q.to(dev), c.k.to(dev), c.v.to(dev), c.dout.to(dev)
    out, lse = ops.gqa_prefill(qd, kd, vd, is_causal=True, scale=c.softmax_scale)
    wants = {}
    for b, h in ((0, 0), (5, 9), (7, 15)):
        sl = (slice(b, b + 1), slice(h, h + 1))
        o_ref, l_ref = orc.cpu_sdpa_forward(c.q[sl], c.k[sl], c.v[sl], causal=True, scale=c.softmax_scale)
        wants[sl] = orc.cpu_sdpa_backward(c.dout[sl], c.q[sl], c.k[sl], c.v[sl], o_ref, l_ref, causal=True, scale=c.softmax_scale)
    for deterministic in (False, True):  # the fused kernel, then the dK/dV + dQ pair
        dq, dk, dv = ops._dense_backward(dd, qd, kd, vd, out, lse, True, c.softmax_scale, deterministic=deterministic)
        assert ops.device_status() == 0
        for sl, want in wants.items():
            check_grads((dq[sl], dk[sl], dv[sl]), want)
            # how the bound was met: where |want| <= 2 the plain 2e-2 must hold; the relative arm is for the few larger
            # values bf16 cannot hold to 2e-2 (at most one element in a thousand may need it)
            for name, g, w in zip(("dq", "dk", "dv"), (dq[sl], dk[sl], dv[sl]), want):
                rep = orc.grad_error_report(g, w)
                print(f"config 3 {name}{tuple((x.start for x in sl))} deterministic={deterministic}: {rep}")
                assert rep["max_abs_where_want_le_2"] <= 2e-2, (name, rep)
                assert rep["beyond_abs_bound"] <= rep["elements"] // 1000, (name, rep)
        dq2, dk2, dv2 = ops._dense_backward(dd * 2, qd, kd, vd, out, lse, True, c.softmax_scale, deterministic=deterministic)
        assert torch.equal(dk2, dk * 2) and torch.equal(dv2, dv * 2)
        if deterministic:
            assert torch.equal(dq2, dq * 2)
        else:  # the order of the fused kernel's dQ reductions varies: equal up to fp32 rounding of the sums
            assert orc.error_stats(dq2, dq.float() * 2)[0] <= 2e-2
        for t in (dq, dk, dv):
            assert torch.isfinite(t.float()).all()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H,Lq,Lk,D,causal", [
    (2, 4, 256, 256, 128, True),
    (1, 2, 113, 203, 128, True),     # the reference sweeps odd Lq != Lk (test_...py:940-946)
    (1, 2, 384, 128, 64, False),
])
def test_reference_tests_own_tolerance_rule(cuda_device, native_lib, dtype, B, H, Lq, Lk, D, causal):
    """Second check with the reference suite's own bar (test_scaled_dot_product_attention.py:1077-1110):
    the kernel may be at most 2x (dq: 4x) as far from the fp32 math as the same math run in the
    low-precision dtype."""
    g = torch.Generator().manual_seed(21)
    q, k, v = (torch.randn(s, generator=g).to(dtype) for s in ((B, H, Lq, D), (B, H, Lk, D), (B, H, Lk, D)))
    dout = torch.rand((B, H, Lq, D), generator=g).to(dtype)
    out, lse, dq, dk, dv = run_fwd_bwd(cuda_device, q, k, v, dout, causal)
    o_true, _ = orc.attention_math(q, k, v, causal=causal)
    o_lp, _ = orc.attention_math(q, k, v, causal=causal, dtype=dtype)
    g_true = orc.attention_math_backward(q, k, v, dout, causal=causal)
    g_lp = orc.attention_math_backward(q, k, v, dout, causal=causal, dtype=dtype)
    orc.assert_close_reference_rule(out, o_true, o_lp, "out")
    orc.assert_close_reference_rule(dq, g_true[0], g_lp[0], "dq", fudge=4)
    orc.assert_close_reference_rule(dk, g_true[1], g_lp[1], "dk")
    orc.assert_close_reference_rule(dv, g_true[2], g_lp[2], "dv")
