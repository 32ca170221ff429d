"""Parity at the full benchmark sizes of the packed varlen GQA configuration (16 sequences, 34 004 tokens,
Hq 32 / Hkv 8, causal) and of the split-KV decode configuration (B 64, Lkv 32 768, 8 GiB of K + V).

The CPU oracle cannot finish those whole tensors in seconds, so each test compares sampled units with the oracle
(whole sequences x KV-head groups; whole batch elements) and adds a property that covers every element:
causality per sequence (perturbing the keys and values at positions >= t leaves rows < t bit-identical) for the
prefill, and independence of the split count for decode.

Tolerances: bf16 outputs and gradients max-abs 2e-2 / mean-abs 2e-3 (gradients: max(2e-2, 1e-2 |want|)), fp32
logsumexp 1e-5.
"""
import pytest
import torch

from oracle import sdpa_oracle as orc
from torch_mlu_b200 import ops, workloads

pytestmark = pytest.mark.gpu

GROUP = 4  # query heads per KV head in the varlen configuration


def _unit(c, seq, kvh):
    """(q [1, 4, L, D], k, v [1, 1, L, D]) of one (sequence, KV head) unit of the packed case."""
    lo, hi = int(c.cu_seqlens[seq]), int(c.cu_seqlens[seq + 1])
    q = c.q[lo:hi, kvh * GROUP:(kvh + 1) * GROUP].transpose(0, 1).unsqueeze(0)
    k = c.k[lo:hi, kvh:kvh + 1].transpose(0, 1).unsqueeze(0)
    v = c.v[lo:hi, kvh:kvh + 1].transpose(0, 1).unsqueeze(0)
    return lo, hi, q, k, v


@pytest.fixture(scope="module")
def config4(cuda_device):
    c = workloads.config4_varlen_gqa()
    assert c.seqlens == workloads.CONFIG4_SEQLENS and sum(c.seqlens) == 34004
    dev = cuda_device
    return c, c.q.to(dev), c.k.to(dev), c.v.to(dev), c.cu_seqlens.to(dev)


def test_config4_forward_full_size(cuda_device, native_lib, config4):
    c, q, k, v, cu = config4
    mx = max(c.seqlens)
    out, lse, *_ = ops._flash_attention_forward(q, k, v, cu, cu, mx, mx, 0.0, True, False, scale=c.softmax_scale)
    assert ops.device_status() == 0
    assert out.shape == (34004, 32, 128) and lse.shape == (32, 34004)
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    # the longest sequence (4038), the shortest (577) and two more whose last 128-row tile is ragged
    # (3277 = 25 * 128 + 77, 925 = 7 * 128 + 29), each on another KV-head group
    for seq, kvh in ((0, 0), (12, 7), (7, 3), (1, 5)):
        lo, hi, qs, ks, vs = _unit(c, seq, kvh)
        o_ref, l_ref = orc.cpu_sdpa_forward(qs, ks, vs, causal=True, scale=c.softmax_scale)
        got_o = out[lo:hi, kvh * GROUP:(kvh + 1) * GROUP].transpose(0, 1).unsqueeze(0)
        got_l = lse[kvh * GROUP:(kvh + 1) * GROUP, lo:hi].unsqueeze(0)
        orc.assert_close_bf16(got_o, o_ref, f"out seq {seq} kv head {kvh}")
        orc.assert_close_lse(got_l, l_ref, f"lse seq {seq} kv head {kvh}")
    # causality, every sequence and head at once: keys / values from the middle of each sequence on are changed
    k2, v2 = k.clone(), v.clone()
    cuts = []
    for i, n in enumerate(c.seqlens):
        t = int(c.cu_seqlens[i]) + n // 2 + 3
        cuts.append(t)
        k2[t:int(c.cu_seqlens[i + 1])] *= -1
        v2[t:int(c.cu_seqlens[i + 1])] = 3.0
    out2, lse2, *_ = ops._flash_attention_forward(q, k2, v2, cu, cu, mx, mx, 0.0, True, False, scale=c.softmax_scale)
    for i, t in enumerate(cuts):
        lo, hi = int(c.cu_seqlens[i]), int(c.cu_seqlens[i + 1])
        assert torch.equal(out[lo:t], out2[lo:t]) and torch.equal(lse[:, lo:t], lse2[:, lo:t]), f"sequence {i}"
        assert not torch.equal(out[t:hi], out2[t:hi]), f"sequence {i}"


def test_config4_backward_full_size(cuda_device, native_lib, config4):
    c, q, k, v, cu = config4
    dev = cuda_device
    mx = max(c.seqlens)
    g = torch.Generator().manual_seed(33)
    dout_h = torch.randn(c.q.shape, generator=g).bfloat16()
    dout = dout_h.to(dev)
    out, lse, *_ = ops._flash_attention_forward(q, k, v, cu, cu, mx, mx, 0.0, True, False, scale=c.softmax_scale)
    e = torch.empty((0,), dtype=torch.int64)
    dq, dk, dv = ops._flash_attention_backward(dout, q, k, v, out, lse, cu, cu, mx, mx, 0.0, True, e, e,
                                               scale=c.softmax_scale)
    assert ops.device_status() == 0
    assert torch.isfinite(dq.float()).all() and torch.isfinite(dk.float()).all() and torch.isfinite(dv.float()).all()
    # one whole sequence over all heads (the shortest), and one KV-head group of the longest
    for seq, kvhs in ((12, range(8)), (0, (2,))):
        for kvh in kvhs:
            lo, hi, qs, ks, vs = _unit(c, seq, kvh)
            ds = dout_h[lo:hi, kvh * GROUP:(kvh + 1) * GROUP].transpose(0, 1).unsqueeze(0)
            o_ref, l_ref = orc.cpu_sdpa_forward(qs, ks, vs, causal=True, scale=c.softmax_scale)
            dq_r, dk_r, dv_r = orc.cpu_sdpa_backward(ds, qs, ks, vs, o_ref, l_ref, causal=True, scale=c.softmax_scale)
            tag = f"seq {seq} kv head {kvh}"
            orc.assert_close_grad_bf16(dq[lo:hi, kvh * GROUP:(kvh + 1) * GROUP].transpose(0, 1).unsqueeze(0), dq_r, "dq " + tag)
            orc.assert_close_grad_bf16(dk[lo:hi, kvh:kvh + 1].transpose(0, 1).unsqueeze(0), dk_r, "dk " + tag)
            orc.assert_close_grad_bf16(dv[lo:hi, kvh:kvh + 1].transpose(0, 1).unsqueeze(0), dv_r, "dv " + tag)
    # linearity in dO on the whole tensors: doubling dO doubles every gradient exactly (powers of two commute with
    # every rounding on the way); the dQ sums of the fused backward are formed in an order that may differ between
    # launches, so dQ is compared at the gradient tolerance instead
    dq2, dk2, dv2 = ops._flash_attention_backward(dout * 2, q, k, v, out, lse, cu, cu, mx, mx, 0.0, True, e, e,
                                                  scale=c.softmax_scale)
    assert torch.equal(dk2, dk * 2) and torch.equal(dv2, dv * 2)
    orc.assert_close_grad_bf16(dq2, dq.float() * 2, "dq linearity")


def test_config5_decode_full_size(cuda_device, native_lib):
    dev = cuda_device
    c = workloads.config5_decode(device=dev)  # drawn per batch element: the host never holds the 8 GiB
    assert c.k.shape == (64, 8, 32768, 128)
    out, lse = ops.decode_attention(c.q, c.k, c.v, scale=c.softmax_scale)
    assert ops.device_status() == 0
    assert out.shape == (64, 32, 1, 128) and lse.shape == (64, 32, 1)
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    for b in (0, 21, 42, 63):
        o_ref, l_ref = orc.cpu_sdpa_forward(c.q[b:b + 1].cpu(), c.k[b:b + 1].cpu(), c.v[b:b + 1].cpu(), scale=c.softmax_scale)
        orc.assert_close_bf16(out[b:b + 1], o_ref, f"out[{b}]")
        orc.assert_close_lse(lse[b:b + 1], l_ref, f"lse[{b}]")
    # every batch element and head: another split count gives the same answer up to the fp32 merge rounding
    o1, l1 = ops.decode_attention(c.q, c.k, c.v, scale=c.softmax_scale, num_splits=5)
    assert orc.error_stats(o1, out)[0] <= 2e-3 and orc.error_stats(l1, lse)[0] <= 2e-6
    # and the kernel reads what it is given: negating V of one batch element negates that element's output only
    c.v[37].neg_()
    o2, l2 = ops.decode_attention(c.q, c.k, c.v, scale=c.softmax_scale)
    assert torch.equal(o2[37], -out[37]) and torch.equal(l2, lse)
    keep = [b for b in range(64) if b != 37]
    assert torch.equal(o2[keep], out[keep])
