"""Dropout: the keep-mask kernel against its CPU restatement (Philox4x32-10), and attention with dropout
against the oracle evaluated with the same mask - the way the reference tests check it, through the mask the
operator returns (test/torch_ops/test_scaled_dot_product_attention.py:1016-1070)."""
import pytest
import torch

from oracle import sdpa_oracle as orc
from torch_mlu_b200 import dropout

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,H,Lq,Lk,p", [(2, 3, 200, 300, 0.22), (1, 2, 129, 1, 0.48), (1, 1, 16, 513, 0.1)])
def test_keep_masks_match_the_cpu_philox(cuda_device, native_lib, B, H, Lq, Lk, p):
    m = dropout.KeepMasks(0x1234567890ABCDEF, (5 << 32) + 77, p, B, H, Lq, Lk, cuda_device)
    want = orc.dropout_keep_mask(0x1234567890ABCDEF, (5 << 32) + 77, p, B, H, Lq, Lk)
    assert not torch.equal(want, orc.dropout_keep_mask(0x1234567890ABCDEF, 77, p, B, H, Lq, Lk))
    assert torch.equal(m.dense().cpu(), want)
    assert torch.equal(m.dense_from_cols().cpu(), want)   # the transposed copy holds the same pattern


def test_keep_rate_and_stream_separation(cuda_device, native_lib):
    B, H, L = 2, 4, 1024
    a = dropout.KeepMasks(1, 0, 0.25, B, H, L, L, cuda_device).dense()
    assert abs(float(a.float().mean()) - 0.75) < 2e-3
    # per head, per row and per column the rate holds too (no stripes)
    assert float((a.float().mean(dim=(2, 3)) - 0.75).abs().max()) < 5e-3
    assert float((a.float().mean(dim=3) - 0.75).abs().max()) < 0.08
    assert float((a.float().mean(dim=2) - 0.75).abs().max()) < 0.08
    b = dropout.KeepMasks(1, 1, 0.25, B, H, L, L, cuda_device).dense()      # next offset
    c = dropout.KeepMasks(2, 0, 0.25, B, H, L, L, cuda_device).dense()      # other seed
    for other in (b, c):
        agree = float((a == other).float().mean())
        assert abs(agree - (0.75 ** 2 + 0.25 ** 2)) < 3e-3                  # independent patterns
    again = dropout.KeepMasks(1, 0, 0.25, B, H, L, L, cuda_device).dense()
    assert torch.equal(a, again)


def attention_with_mask(q, k, v, keep, dropout_p, causal, scale=None):
    """fp32 attention with a given dropout pattern: softmax first, then the kept probabilities scaled by
    1 / (1 - p) (attention_ref, test_scaled_dot_product_attention.py:149-160). Bottom-right causal."""
    qf, kf, vf = q.float(), k.float(), v.float()
    sc = orc.calculate_scale(q.shape[-1], scale)
    scores = torch.einsum("bhtd,bhsd->bhts", qf * sc, kf)
    if causal:
        scores = scores.masked_fill(orc.causal_mask_bottom_right(q.shape[2], k.shape[2]), float("-inf"))
    lse = torch.logsumexp(scores, dim=-1)
    attn = torch.softmax(scores, dim=-1)
    dead = torch.isinf(lse) & (lse < 0)
    attn = attn.masked_fill(dead.unsqueeze(-1), 0.0)
    attn = attn.masked_fill(~keep, 0.0) / (1.0 - dropout_p)
    return torch.einsum("bhts,bhsd->bhtd", attn, vf), lse.masked_fill(dead, float("inf"))


def rand(shape, seed, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g).to(dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H,Lq,Lk,D,causal,p", [
    (2, 4, 512, 512, 128, True, 0.22),      # the reference sweeps dropout_p 0.22 and 0.48 (test_...py:945)
    (1, 2, 200, 333, 128, False, 0.48),
    (1, 3, 300, 130, 64, True, 0.22),
    (2, 2, 129, 257, 96, False, 0.1),
])
def test_forward_with_dropout_matches_oracle_with_the_returned_mask(cuda_device, native_lib, dtype, B, H, Lq, Lk, D, causal, p):
    from torch_mlu_b200 import ops
    dev = cuda_device
    q, k, v = rand((B, H, Lq, D), 1, dtype), rand((B, H, Lk, D), 2, dtype), rand((B, H, Lk, D), 3, dtype)
    out, lse, _, _, _, _, seed, offset, debug = ops._scaled_dot_product_flash_attention(q.to(dev), k.to(dev), v.to(dev), p, causal, True)
    assert ops.device_status() == 0
    assert tuple(debug.shape) == (B, H, Lq, Lk) and seed.numel() == 1 and offset.numel() == 1
    keep = (debug > 0).cpu()
    # (tiles the causal mask hides completely carry zeros instead of random bits)
    visible = ~orc.causal_mask_bottom_right(Lq, Lk) if causal else torch.ones(Lq, Lk, dtype=torch.bool)
    assert torch.equal(keep & visible, orc.dropout_keep_mask(int(seed), int(offset), p, B, H, Lq, Lk) & visible)
    o_ref, l_ref = attention_with_mask(q, k, v, keep, p, causal)
    orc.assert_close_bf16(out, o_ref, "out")
    orc.assert_close_lse(lse[..., :Lq], l_ref)        # dropout does not touch the logsumexp
    # a second call draws another pattern
    *_, off2, _ = ops._scaled_dot_product_flash_attention(q.to(dev), k.to(dev), v.to(dev), p, causal, False)
    assert int(off2) != int(offset)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H,Lq,Lk,D,causal,p", [
    (2, 4, 512, 512, 128, True, 0.22),
    (1, 2, 200, 333, 128, False, 0.48),
    (1, 3, 300, 130, 64, True, 0.22),
    (2, 2, 129, 257, 96, False, 0.1),
])
def test_backward_with_dropout_replays_the_pattern(cuda_device, native_lib, dtype, B, H, Lq, Lk, D, causal, p):
    """Gradients against autograd through the fp32 math with the forward's mask (what the reference tests do,
    test_scaled_dot_product_attention.py:1070-1110), held to that suite's own tolerance rule."""
    from torch_mlu_b200 import ops
    dev = cuda_device
    q, k, v = rand((B, H, Lq, D), 1, dtype), rand((B, H, Lk, D), 2, dtype), rand((B, H, Lk, D), 3, dtype)
    dout = torch.rand((B, H, Lq, D), generator=torch.Generator().manual_seed(4)).to(dtype)
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    out, lse, cq, ck, mq, mk, seed, offset, debug = ops._scaled_dot_product_flash_attention(qd, kd, vd, p, causal, True)
    dq, dk, dv = ops._scaled_dot_product_flash_attention_backward(dout.to(dev), qd, kd, vd, out, lse, cq, ck, mq, mk, p, causal,
                                                                  seed, offset)
    assert ops.device_status() == 0
    keep = (debug > 0).cpu()

    def grads(compute_dtype):
        qf, kf, vf = (t.to(compute_dtype).detach().requires_grad_(True) for t in (q, k, v))
        sc = orc.calculate_scale(D, None)
        scores = torch.einsum("bhtd,bhsd->bhts", qf * sc, kf)
        if causal:
            scores = scores.masked_fill(orc.causal_mask_bottom_right(Lq, Lk), float("-inf"))
        attn = torch.softmax(scores, dim=-1)
        dead = torch.isinf(torch.logsumexp(scores.float(), dim=-1))
        attn = attn.masked_fill(dead.unsqueeze(-1), 0.0).masked_fill(~keep, 0.0) / (1.0 - p)
        o = torch.einsum("bhts,bhsd->bhtd", attn, vf)
        o.backward(dout.to(compute_dtype))
        return o.detach(), qf.grad, kf.grad, vf.grad

    true, lowp = grads(torch.float32), grads(dtype)
    orc.assert_close_reference_rule(out, true[0], lowp[0], "out")
    orc.assert_close_reference_rule(dq, true[1], lowp[1], "dq", fudge=4)
    orc.assert_close_reference_rule(dk, true[2], lowp[2], "dk")
    orc.assert_close_reference_rule(dv, true[3], lowp[3], "dv")
    # and the absolute tolerances of the other parity tests where gradients are of order one
    orc.assert_close_grad_bf16(dq, true[1], "dq")
    orc.assert_close_grad_bf16(dk, true[2], "dk")
    orc.assert_close_grad_bf16(dv, true[3], "dv")


def test_causal_masks_skip_hidden_tiles_only(cuda_device, native_lib):
    B, H, Lq, Lk, p = 1, 2, 300, 520, 0.3
    full = dropout.KeepMasks(9, 5, p, B, H, Lq, Lk, cuda_device).dense().cpu()
    causal = dropout.KeepMasks(9, 5, p, B, H, Lq, Lk, cuda_device, True).dense().cpu()
    visible = ~orc.causal_mask_bottom_right(Lq, Lk)
    assert torch.equal(full & visible, causal & visible)
    assert not bool((causal & ~visible)[..., :128, 384 + 128:].any())     # a tile above the diagonal: zeros


def test_manual_seed_repeats_the_pattern(cuda_device, native_lib):
    from torch_mlu_b200 import ops
    q = rand((1, 2, 256, 128), 1).to(cuda_device)
    torch.cuda.manual_seed(77)
    a = ops._scaled_dot_product_flash_attention(q, q, q, 0.3, True, False)
    b = ops._scaled_dot_product_flash_attention(q, q, q, 0.3, True, False)
    torch.cuda.manual_seed(77)
    c = ops._scaled_dot_product_flash_attention(q, q, q, 0.3, True, False)
    assert int(a[7]) != int(b[7]) and not torch.equal(a[0], b[0])
    assert int(a[6]) == int(c[6]) and int(a[7]) == int(c[7]) and torch.equal(a[0], c[0])


@pytest.mark.parametrize("lens_q,lens_k,Hq,Hkv,causal,p", [
    ([100, 300, 257], [100, 300, 257], 4, 2, True, 0.22),
    ([512, 64, 130], [200, 333, 130], 2, 2, False, 0.48),
    ([1, 129, 255], [70, 129, 400], 4, 1, True, 0.1),
])
def test_packed_varlen_forward_and_backward_with_dropout(cuda_device, native_lib, lens_q, lens_k, Hq, Hkv, causal, p):
    """_flash_attention_forward / _backward with dropout_p > 0 (the path the reference's dense wrapper runs on,
    FlashAttention_internal.cpp:57-267): every sequence against fp32 math with the returned pattern, whose bits are
    those of the dense operator for the same batch index."""
    from torch_mlu_b200 import ops
    dev = cuda_device
    D = 128
    cu_q, cu_k = [0], [0]
    for a, b in zip(lens_q, lens_k):
        cu_q.append(cu_q[-1] + a)
        cu_k.append(cu_k[-1] + b)
    q, k, v = rand((cu_q[-1], Hq, D), 1), rand((cu_k[-1], Hkv, D), 2), rand((cu_k[-1], Hkv, D), 3)
    dout = torch.rand((cu_q[-1], Hq, D), generator=torch.Generator().manual_seed(4)).bfloat16()
    cq, ck = (torch.tensor(c, dtype=torch.int32, device=dev) for c in (cu_q, cu_k))
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    out, lse, seed, offset, debug = ops._flash_attention_forward(qd, kd, vd, cq, ck, max(lens_q), max(lens_k), p, causal, True)
    dq, dk, dv = ops._flash_attention_backward(dout.to(dev), qd, kd, vd, out, lse, cq, ck, max(lens_q), max(lens_k), p, causal,
                                               seed, offset)
    assert ops.device_status() == 0
    B = len(lens_q)
    assert tuple(debug.shape) == (B, Hq, max(lens_q), max(lens_k))
    g = Hq // Hkv
    for b in range(B):
        lq, lk = lens_q[b], lens_k[b]
        sq, sk = slice(cu_q[b], cu_q[b + 1]), slice(cu_k[b], cu_k[b + 1])
        keep = (debug[b, :, :lq, :lk] > 0).cpu().unsqueeze(0)
        visible = ~orc.causal_mask_bottom_right(lq, lk) if causal else torch.ones(lq, lk, dtype=torch.bool)
        want_bits = orc.dropout_keep_mask(int(seed), int(offset), p, B, Hq, lq, lk)[b:b + 1]
        assert torch.equal(keep & visible, want_bits & visible), f"sequence {b}"
        one = lambda x, sl: x[sl].transpose(0, 1).unsqueeze(0)

        def run(dtype):
            qf, kf, vf = (one(t, s).to(dtype).detach().requires_grad_(True) for t, s in ((q, sq), (k, sk), (v, sk)))
            scores = torch.einsum("bhtd,bhsd->bhts", qf * D ** -0.5, kf.repeat_interleave(g, dim=1))
            if causal:
                scores = scores.masked_fill(~visible, float("-inf"))
            dead = torch.isinf(torch.logsumexp(scores.float(), dim=-1))
            attn = torch.softmax(scores, dim=-1).masked_fill(dead.unsqueeze(-1), 0.0).masked_fill(~keep, 0.0) / (1 - p)
            o = torch.einsum("bhts,bhsd->bhtd", attn, vf.repeat_interleave(g, dim=1))
            o.backward(one(dout, sq).to(dtype))
            return o.detach(), qf.grad, kf.grad, vf.grad

        true, lowp = run(torch.float32), run(torch.bfloat16)
        orc.assert_close_bf16(one(out, sq), true[0], f"out[{b}]")
        for name, got, i, fudge in (("dq", one(dq, sq), 1, 4), ("dk", one(dk, sk), 2, 2), ("dv", one(dv, sk), 3, 2)):
            orc.assert_close_reference_rule(got, true[i], lowp[i], f"{name}[{b}]", fudge=fudge)


from test_oracle import DROPOUT_GOLDEN, load_dropout_golden  # noqa: E402


@pytest.mark.parametrize("path", DROPOUT_GOLDEN, ids=lambda p: p.split("dropout_ref_")[-1][:-4])
def test_kernels_with_dropout_match_reference_golden(cuda_device, native_lib, path):
    """Forward and backward with the golden file's Philox pair against what the reference's attention_ref gave
    for the same pattern (GQA included: the kernels reduce dK/dV over the group)."""
    from torch_mlu_b200 import ops
    dev = cuda_device
    g = load_dropout_golden(path)
    B, H, Lq, Lk = g["keep"].shape
    q, k, v, do = (g[n].to(dev) for n in ("q", "k", "v", "dout"))
    keep = dropout.KeepMasks(g["seed"], g["offset"], g["p"], B, H, Lq, Lk, dev, g["causal"])
    sc = ops.calculate_scale(q, None)
    out, lse = ops._dense_forward(q, k, v, g["causal"], sc, allow_gqa=True, kernel=1, keep=keep)
    dq, dk, dv = ops._dense_backward(do, q, k, v, out, lse, g["causal"], sc, keep=keep)
    assert ops.device_status() == 0
    orc.assert_close_bf16(out, g["out"], "out")
    orc.assert_close_grad_bf16(dq, g["dq"], "dq")
    orc.assert_close_grad_bf16(dk, g["dk"], "dk")
    orc.assert_close_grad_bf16(dv, g["dv"], "dv")
