"""Out-of-bounds write checks: every output of every kernel is a view inside a larger NaN-filled buffer, and after
the call each NaN outside the view is still there while the view itself matches the oracle.

The bands sit where an off-by-one would land: rows before and after each batch element's sequence (tiles clipped
by a tensor map, row-wise stores of ragged packed tiles), columns past head_dim in every row (head dims that run in
a wider kernel instance), and words before and after the contiguous logsumexp. This is the stand-in for a memory
checker run, which the GPUs these tests run on do not offer.
"""
import ctypes

import pytest
import torch

from oracle import sdpa_oracle as orc
from torch_mlu_b200 import _cabi, ops

pytestmark = pytest.mark.gpu

NAN = float("nan")
ROW_PAD, COL_PAD, FLAT_PAD = 2, 8, 64


def rand(shape, seed, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g).to(dtype)


class Banded:
    """A [B, H, L, D] (dense) or [T, H, D] (packed) tensor placed inside a NaN-filled buffer with ROW_PAD spare rows
    on both sides of the row axis and COL_PAD spare columns behind every row."""

    def __init__(self, shape, dev, dtype=torch.bfloat16, fill=NAN):
        self.packed = len(shape) == 3
        if self.packed:
            T, H, D = shape
            self.buf = torch.full((T + 2 * ROW_PAD, H, D + COL_PAD), NAN, dtype=dtype, device=dev)
            self.inner = self.buf[ROW_PAD:ROW_PAD + T, :, :D]
            self.view = self.inner
        else:
            B, H, L, D = shape
            self.buf = torch.full((B, L + 2 * ROW_PAD, H, D + COL_PAD), NAN, dtype=dtype, device=dev)
            self.inner = self.buf[:, ROW_PAD:ROW_PAD + L, :, :D]
            self.view = self.inner.transpose(1, 2)
        if fill == fill:  # not NaN: the call expects a cleared buffer
            self.inner.fill_(fill)

    def assert_bands_intact(self, name):
        nans = int(torch.isnan(self.buf).sum())
        inside = int(torch.isnan(self.inner).sum())
        assert inside == 0, f"{name}: {inside} elements of the output were never written"
        assert nans == self.buf.numel() - self.inner.numel(), \
            f"{name}: {self.buf.numel() - self.inner.numel() - nans} guard elements were overwritten"


class BandedFlat:
    """A contiguous fp32 tensor with FLAT_PAD NaN words before and after it."""

    def __init__(self, shape, dev):
        n = 1
        for s in shape:
            n *= s
        self.buf = torch.full((n + 2 * FLAT_PAD,), NAN, dtype=torch.float32, device=dev)
        self.view = self.buf[FLAT_PAD:FLAT_PAD + n].view(shape)

    def assert_bands_intact(self, name):
        assert torch.isnan(self.buf[:FLAT_PAD]).all() and torch.isnan(self.buf[-FLAT_PAD:]).all(), \
            f"{name}: words next to the tensor were overwritten"
        assert not torch.isnan(self.view).any(), f"{name}: elements of the output were never written"


def set_bwd(p, dout, dq, dk, dv, packed):
    p.dout, p.dq, p.dk, p.dv = dout.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    setter = ops._set_strides_thd if packed else ops._set_strides_bhld
    for name, t in (("do", dout), ("dq", dq), ("dk", dk), ("dv", dv)):
        setter(p, name, t)


@pytest.mark.parametrize("B,Hq,Hkv,Lq,Lk,D,causal", [
    (2, 4, 2, 200, 200, 128, True),    # Lq % 128 != 0: the last tile's stores are clipped
    (1, 2, 2, 333, 130, 80, False),    # head_dim 80 runs in the 128-column kernel: columns 80.. are clipped
    (1, 2, 1, 129, 257, 64, True),
    (2, 2, 2, 1, 300, 128, False),     # one query row: the tile kernel's smallest case
    (1, 4, 2, 200, 333, 160, True),    # head dims above 128: the kernels that stage 256-column tiles
    (2, 2, 1, 129, 70, 256, False),
])
def test_dense_forward_and_backward_write_nothing_outside_their_outputs(cuda_device, native_lib, B, Hq, Hkv, Lq, Lk, D, causal):
    dev = cuda_device
    q, k, v, dout = rand((B, Hq, Lq, D), 1), rand((B, Hkv, Lk, D), 2), rand((B, Hkv, Lk, D), 3), rand((B, Hq, Lq, D), 4)
    qd, kd, vd, dd = q.to(dev), k.to(dev), v.to(dev), dout.to(dev)
    out, lse = Banded((B, Hq, Lq, D), dev), BandedFlat((B, Hq, Lq), dev)
    scale = D ** -0.5
    p = ops._dense_params(qd, kd, vd, out.view, lse.view, causal, scale, _cabi.KERNEL_PREFILL)
    ops._run_fwd(p, dev)
    assert ops.device_status() == 0
    out.assert_bands_intact("out")
    lse.assert_bands_intact("lse")
    o_ref, l_ref = orc.cpu_sdpa_forward(q, k, v, causal=causal)
    orc.assert_close_bf16(out.view, o_ref, "out")
    orc.assert_close_lse(lse.view, l_ref)

    dq, dk, dv = Banded((B, Hq, Lq, D), dev), Banded((B, Hkv, Lk, D), dev), Banded((B, Hkv, Lk, D), dev)
    for deterministic in (0, 1):
        for t in (dq, dk, dv):
            t.inner.fill_(NAN)
        p = ops._dense_params(qd, kd, vd, out.view, lse.view, causal, scale)
        set_bwd(p, dd, dq.view, dk.view, dv.view, packed=False)
        p.deterministic = deterministic
        ops._run_bwd(p, dev)
        assert ops.device_status() == 0
        dq_r, dk_r, dv_r = orc.cpu_sdpa_backward(dout, q, k, v, o_ref, l_ref, causal=causal)
        for name, t, want in (("dq", dq, dq_r), ("dk", dk, dk_r), ("dv", dv, dv_r)):
            t.assert_bands_intact(f"{name} (deterministic={deterministic})")
            orc.assert_close_grad_bf16(t.view, want, name)


@pytest.mark.parametrize("lens,Hq,Hkv,D,causal", [
    ([130, 70, 1, 255], 4, 2, 128, True),   # every sequence ends inside a tile: row-wise stores next to a neighbour
    ([128, 129, 127], 2, 2, 64, False),
    ([300, 45], 8, 2, 96, True),
    ([130, 70, 1, 255], 4, 2, 256, True),
    ([128, 129], 2, 2, 136, False),
])
def test_packed_forward_and_backward_write_nothing_outside_their_outputs(cuda_device, native_lib, lens, Hq, Hkv, D, causal):
    dev = cuda_device
    total = sum(lens)
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    q, k, v, dout = rand((total, Hq, D), 1), rand((total, Hkv, D), 2), rand((total, Hkv, D), 3), rand((total, Hq, D), 4)
    qd, kd, vd, dd = q.to(dev), k.to(dev), v.to(dev), dout.to(dev)
    out, lse = Banded((total, Hq, D), dev), BandedFlat((Hq, total), dev)
    scale = D ** -0.5
    p = ops._varlen_params(qd, kd, vd, out.view, lse.view, cu_t, cu_t, max(lens), max(lens), causal, scale)
    ops._run_fwd(p, dev)
    assert ops.device_status() == 0
    out.assert_bands_intact("out")
    lse.assert_bands_intact("lse")
    o_ref, l_ref = orc.varlen_forward(q, k, v, cu, cu, causal=causal)
    orc.assert_close_bf16(out.view, o_ref, "out")
    orc.assert_close_lse(lse.view, l_ref)

    dq, dk, dv = Banded((total, Hq, D), dev), Banded((total, Hkv, D), dev), Banded((total, Hkv, D), dev)
    dq_r, dk_r, dv_r = orc.varlen_backward(dout, q, k, v, cu, cu, causal=causal)
    for deterministic in (0, 1):
        for t in (dq, dk, dv):
            t.inner.fill_(NAN)
        p = ops._varlen_params(qd, kd, vd, out.view, lse.view, cu_t, cu_t, max(lens), max(lens), causal, scale)
        set_bwd(p, dd, dq.view, dk.view, dv.view, packed=True)
        p.deterministic = deterministic
        ops._run_bwd(p, dev)
        assert ops.device_status() == 0
        for name, t, want in (("dq", dq, dq_r), ("dk", dk, dk_r), ("dv", dv, dv_r)):
            t.assert_bands_intact(f"{name} (deterministic={deterministic})")
            orc.assert_close_grad_bf16(t.view, want, name)


def test_bias_gradient_stays_inside_its_buffer(cuda_device, native_lib):
    """grad_bias rows are written 8 keys at a time up to seqlen_k rounded up to 8; nothing beyond that, and no row
    outside [0, seqlen_q)."""
    dev = cuda_device
    B, H, Lq, Lk, D = 1, 2, 150, 203, 128
    lk8 = (Lk + 7) // 8 * 8
    q, k, v, dout = rand((B, H, Lq, D), 1), rand((B, H, Lk, D), 2), rand((B, H, Lk, D), 3), rand((B, H, Lq, D), 4)
    bias_h = rand((B, H, Lq, Lk), 5)
    qd, kd, vd, dd = q.to(dev), k.to(dev), v.to(dev), dout.to(dev)
    bias = ops._prepare_bias(bias_h.to(dev), qd, kd)
    out, lse = ops._dense_forward(qd, kd, vd, False, D ** -0.5, allow_gqa=False, bias=bias)
    buf = torch.full((B, H, Lq + 2 * ROW_PAD, lk8 + COL_PAD), NAN, dtype=torch.bfloat16, device=dev)
    inner = buf[:, :, ROW_PAD:ROW_PAD + Lq, :lk8]
    inner.zero_()
    dq, dk, dv = ops._dense_backward(dd, qd, kd, vd, out, lse, False, D ** -0.5, bias=bias, dbias=inner[..., :Lk])
    assert ops.device_status() == 0
    assert int(torch.isnan(buf).sum()) == buf.numel() - inner.numel() and not torch.isnan(inner).any()
    # and it is the gradient: dS of fp32 math with the same bias
    s = torch.einsum("bhqd,bhkd->bhqk", q.float(), k.float()) * D ** -0.5 + bias_h.float()
    pr = torch.softmax(s, dim=-1)
    dp = torch.einsum("bhqd,bhkd->bhqk", dout.float(), v.float())
    ds = pr * (dp - (dp * pr).sum(-1, keepdim=True))
    orc.assert_close_grad_bf16(inner[..., :Lk], ds, "dbias")


@pytest.mark.parametrize("D,splits", [(128, 1), (128, 6), (64, 4)])
def test_decode_writes_nothing_outside_its_outputs(cuda_device, native_lib, D, splits):
    dev = cuda_device
    B, Hq, Hkv, Lk = 3, 8, 2, 1111
    q, k, v = rand((B, Hq, 1, D), 1), rand((B, Hkv, Lk, D), 2), rand((B, Hkv, Lk, D), 3)
    out, lse = Banded((B, Hq, 1, D), dev), BandedFlat((B, Hq, 1), dev)
    p = ops._dense_params(q.to(dev), k.to(dev), v.to(dev), out.view, lse.view, False, D ** -0.5, _cabi.KERNEL_DECODE, splits)
    ops._run_fwd(p, dev)
    assert ops.device_status() == 0
    out.assert_bands_intact("decode out")
    lse.assert_bands_intact("decode lse")
    o_ref, l_ref = orc.cpu_sdpa_forward(q, k, v)
    orc.assert_close_bf16(out.view, o_ref, "decode out")
    orc.assert_close_lse(lse.view, l_ref)
    # the entry point that keeps its split partials in the library's own array
    out2, lse2 = Banded((B, Hq, 1, D), dev), BandedFlat((B, Hq, 1), dev)
    p = ops._dense_params(q.to(dev), k.to(dev), v.to(dev), out2.view, lse2.view, False, D ** -0.5, _cabi.KERNEL_DECODE, splits)
    _cabi.check(native_lib.sdpa_b200_decode_static(ctypes.byref(p), torch.cuda.current_stream().cuda_stream), "decode_static")
    torch.cuda.synchronize()
    out2.assert_bands_intact("decode_static out")
    lse2.assert_bands_intact("decode_static lse")
    assert torch.equal(out2.view, out.view) and torch.equal(lse2.view, lse.view)
