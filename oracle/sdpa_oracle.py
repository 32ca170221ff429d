"""CPU oracle for the attention hot path. TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference arm may import
this module, and only as the checker or the timed CPU baseline - never as the product path.

Two independent statements of the same math, both fp32 (or fp64 on request) on the CPU:

* ``attention_math``: the explicit einsum/softmax formulation of the reference's own test
  oracle ``attention_ref`` (test/torch_ops/test_scaled_dot_product_attention.py:78-161) with its
  bottom-right-aligned causal mask ``construct_local_mask`` (:46-75, rule at :69), GQA head
  repeat (:119-120) and scale handling (:122-126, default 1/sqrt(d) as sdp_utils.h:40-47).
  Additionally returns logsumexp as mha_varlen_fwd defines it (natural log of the row sums of
  exp(scale*QK^T), FlashAttention_internal.cpp:129, 261-265).
* ``cpu_sdpa_forward/backward``: torch's CPU fused SDPA
  (aten::_scaled_dot_product_flash_attention_for_cpu[_backward]) in fp32 - the path the task
  names as the reference implementation runnable on the host.

Parity pins: ``attention_math`` is checked against golden vectors produced by executing the
reference's ``attention_ref`` source (tests/golden/make_golden.py, tests/test_oracle.py).
The reference pins O, dQ, dK, dV; it never checks logsumexp values, ragged varlen, GQA or
decode - for those the parity of this oracle is unpinned by the reference and rests on the
agreement of the two statements above plus the plain-C restatement in oracle/sdpa_ref.c.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch

NEG_INF = float("-inf")


def calculate_scale(head_dim: int, scale: Optional[float]) -> float:
    """sdp_utils.h:40-47."""
    return float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)


def causal_mask_bottom_right(seqlen_q: int, seqlen_k: int) -> torch.Tensor:
    """True where key j is HIDDEN from query i: j > i + seqlen_k - seqlen_q
    (construct_local_mask with window (-1, 0), test_scaled_dot_product_attention.py:69)."""
    row = torch.arange(seqlen_q).unsqueeze(1)
    col = torch.arange(seqlen_k).unsqueeze(0)
    return col > row + (seqlen_k - seqlen_q)


def attention_math(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool = False,
                   scale: Optional[float] = None, dtype: torch.dtype = torch.float32,
                   keep: Optional[torch.Tensor] = None, dropout_p: float = 0.0
                   ) -> Tuple[torch.Tensor, torch.Tensor]:
    """q [B,Hq,Lq,D], k/v [B,Hkv,Lk,D] -> (out [B,Hq,Lq,D], lse [B,Hq,Lq]) in ``dtype``.

    Fully masked rows give out = 0 (attention_ref, :143-147) and lse = +inf. ``keep`` (bool [B,Hq,Lq,Lk],
    True = kept) with ``dropout_p`` applies dropout after the softmax: dropped probabilities become 0 and the
    rest is scaled by 1 / (1 - dropout_p) (attention_ref, :153-158); the logsumexp is not affected.
    """
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    g = q.shape[1] // k.shape[1]
    if g > 1:
        k = k.repeat_interleave(g, dim=1)
        v = v.repeat_interleave(g, dim=1)
    sc = calculate_scale(q.shape[-1], scale)
    scores = torch.einsum("bhtd,bhsd->bhts", q * sc, k)
    if causal:
        hidden = causal_mask_bottom_right(q.shape[2], k.shape[2])
        scores = scores.masked_fill(hidden, NEG_INF)
    lse = torch.logsumexp(scores, dim=-1)
    attn = torch.softmax(scores, dim=-1)
    dead = torch.isinf(lse) & (lse < 0)
    if dead.any():
        attn = attn.masked_fill(dead.unsqueeze(-1), 0.0)
        lse = lse.masked_fill(dead, float("inf"))
    if keep is not None:
        attn = attn.masked_fill(~keep, 0.0) / (1.0 - dropout_p)
    out = torch.einsum("bhts,bhsd->bhtd", attn, v)
    return out, lse


def attention_math_backward(q, k, v, dout, *, causal=False, scale=None, dtype=torch.float32, keep=None, dropout_p=0.0):
    """Gradients of ``attention_math`` by autograd (what the reference tests do with
    out.backward, test_scaled_dot_product_attention.py:1018-1075). dk/dv come back with Hkv
    heads (the group is summed)."""
    q = q.to(dtype).detach().requires_grad_(True)
    k = k.to(dtype).detach().requires_grad_(True)
    v = v.to(dtype).detach().requires_grad_(True)
    out, _ = attention_math(q, k, v, causal=causal, scale=scale, dtype=dtype, keep=keep, dropout_p=dropout_p)
    out.backward(dout.to(dtype))
    return q.grad, k.grad, v.grad


# --------------------------------------------------------------------------------------
# torch CPU fused SDPA (fp32)
# --------------------------------------------------------------------------------------
def _expand_kv(q, k, v):
    g = q.shape[1] // k.shape[1]
    if g > 1:
        k = k.repeat_interleave(g, dim=1)
        v = v.repeat_interleave(g, dim=1)
    return k, v, g


def _additive_causal(seqlen_q: int, seqlen_k: int) -> torch.Tensor:
    m = torch.zeros(seqlen_q, seqlen_k, dtype=torch.float32)
    return m.masked_fill(causal_mask_bottom_right(seqlen_q, seqlen_k), NEG_INF)


def cpu_sdpa_forward(q, k, v, *, causal=False, scale=None):
    """fp32 torch-CPU SDPA: (out [B,Hq,Lq,D], lse [B,Hq,Lq]).

    torch's CPU kernel aligns ``is_causal`` top-left; for Lq != Lk the bottom-right rule is
    passed as an explicit additive mask instead. Rows with no visible key are patched to the
    library convention (out 0, lse +inf)."""
    q, k, v = q.float().contiguous(), k.float().contiguous(), v.float().contiguous()
    k, v, _ = _expand_kv(q, k, v)
    sc = calculate_scale(q.shape[-1], scale)
    lq, lk = q.shape[2], k.shape[2]
    if causal and lq != lk:
        out, lse = torch.ops.aten._scaled_dot_product_flash_attention_for_cpu(
            q, k, v, 0.0, False, attn_mask=_additive_causal(lq, lk), scale=sc)
        if lq > lk:
            dead = torch.arange(lq) < (lq - lk)
            out = out.clone()
            lse = lse.clone()
            out[:, :, dead] = 0.0
            lse[:, :, dead] = float("inf")
    else:
        out, lse = torch.ops.aten._scaled_dot_product_flash_attention_for_cpu(
            q, k, v, 0.0, bool(causal), attn_mask=None, scale=sc)
    return out, lse


def cpu_sdpa_backward(dout, q, k, v, out, lse, *, causal=False, scale=None):
    """fp32 torch-CPU SDPA backward: (dq [B,Hq,..], dk, dv [B,Hkv,..])."""
    q, k, v = q.float().contiguous(), k.float().contiguous(), v.float().contiguous()
    hkv = k.shape[1]
    k, v, g = _expand_kv(q, k, v)
    sc = calculate_scale(q.shape[-1], scale)
    lq, lk = q.shape[2], k.shape[2]
    mask = None
    is_causal = bool(causal)
    if causal and lq != lk:
        mask = _additive_causal(lq, lk)
        is_causal = False
        if lq > lk:  # keep the dead rows out of the backward's exp(s - lse)
            lse = lse.clone()
            lse[:, :, : lq - lk] = float("inf")
    dq, dk, dv = torch.ops.aten._scaled_dot_product_flash_attention_for_cpu_backward(
        dout.float().contiguous(), q, k, v, out.float().contiguous(), lse.float().contiguous(), 0.0, is_causal,
        attn_mask=mask, scale=sc)
    if g > 1:
        b, _, _, d = dk.shape
        dk = dk.reshape(b, hkv, g, lk, d).sum(2)
        dv = dv.reshape(b, hkv, g, lk, d).sum(2)
    return dq, dk, dv


# --------------------------------------------------------------------------------------
# packed varlen: loop over sequences (layout of FlashAttention_internal.cpp:81-84,112-127)
# --------------------------------------------------------------------------------------
def varlen_forward(q, k, v, cu_q: Sequence[int], cu_k: Sequence[int], *, causal=False, scale=None,
                   impl=cpu_sdpa_forward):
    """q [total_q,Hq,D], k/v [total_k,Hkv,D] -> (out [total_q,Hq,D] fp32, lse [Hq,total_q] fp32)."""
    outs: List[torch.Tensor] = []
    lses: List[torch.Tensor] = []
    for i in range(len(cu_q) - 1):
        qs = q[cu_q[i]:cu_q[i + 1]].transpose(0, 1).unsqueeze(0)
        ks = k[cu_k[i]:cu_k[i + 1]].transpose(0, 1).unsqueeze(0)
        vs = v[cu_k[i]:cu_k[i + 1]].transpose(0, 1).unsqueeze(0)
        o, l = impl(qs, ks, vs, causal=causal, scale=scale)
        outs.append(o[0].transpose(0, 1))
        lses.append(l[0])
    return torch.cat(outs, 0), torch.cat(lses, 1)


def varlen_backward(dout, q, k, v, cu_q, cu_k, *, causal=False, scale=None):
    """(dq [total_q,Hq,D], dk, dv [total_k,Hkv,D]) fp32, per-sequence CPU SDPA backward."""
    dqs, dks, dvs = [], [], []
    for i in range(len(cu_q) - 1):
        sl_q = slice(cu_q[i], cu_q[i + 1])
        sl_k = slice(cu_k[i], cu_k[i + 1])
        qs = q[sl_q].transpose(0, 1).unsqueeze(0)
        ks = k[sl_k].transpose(0, 1).unsqueeze(0)
        vs = v[sl_k].transpose(0, 1).unsqueeze(0)
        ds = dout[sl_q].transpose(0, 1).unsqueeze(0)
        o, l = cpu_sdpa_forward(qs, ks, vs, causal=causal, scale=scale)
        dq, dk, dv = cpu_sdpa_backward(ds, qs, ks, vs, o, l, causal=causal, scale=scale)
        dqs.append(dq[0].transpose(0, 1))
        dks.append(dk[0].transpose(0, 1))
        dvs.append(dv[0].transpose(0, 1))
    return torch.cat(dqs, 0), torch.cat(dks, 0), torch.cat(dvs, 0)


# --------------------------------------------------------------------------------------
# comparison helpers (tolerances named by the task: bf16 outputs/gradients max-abs 2e-2 and
# mean-abs 2e-3; fp32 logsumexp 1e-5)
# --------------------------------------------------------------------------------------
BF16_MAX_ABS = 2e-2
BF16_MEAN_ABS = 2e-3
LSE_MAX_ABS = 1e-5


def error_stats(got: torch.Tensor, want: torch.Tensor) -> Tuple[float, float]:
    d = (got.detach().float().cpu() - want.detach().float().cpu()).abs()
    return float(d.max()), float(d.mean())


def assert_close_bf16(got, want, name: str, max_abs: float = BF16_MAX_ABS, mean_abs: float = BF16_MEAN_ABS):
    mx, mean = error_stats(got, want)
    assert math.isfinite(mx), f"{name}: non-finite values"
    assert mx <= max_abs and mean <= mean_abs, f"{name}: max-abs {mx:.3e} (limit {max_abs}), mean-abs {mean:.3e} (limit {mean_abs})"
    return mx, mean


def assert_close_grad_bf16(got, want, name: str, max_abs: float = BF16_MAX_ABS, mean_abs: float = BF16_MEAN_ABS,
                           rel_large: float = 1e-2):
    """Gradient check: every element within max(2e-2, 1e-2*|want|) and mean-abs within 2e-3.

    The absolute bound alone cannot hold for large gradient values in bf16: one ulp is 0.0156
    for |x| in [2,4) and 0.031 in [4,8) (summed GQA dK/dV reach that), so rounding the exact
    answer to the output dtype already spends most of 2e-2. The relative arm (1e-2) is tighter
    than the reference tests' own bf16 rule (rtol 1.6e-2 with a fudge factor of 2 or more,
    test/torch_ops/test_scaled_dot_product_attention.py:166-167, 188-204, 1079-1082)."""
    g = got.detach().float().cpu()
    w = want.detach().float().cpu()
    d = (g - w).abs()
    assert torch.isfinite(d).all(), f"{name}: non-finite values"
    bound = torch.clamp(w.abs() * rel_large, min=max_abs)
    worst = float((d - bound).max())
    assert worst <= 0.0, f"{name}: exceeds max({max_abs}, {rel_large}*|want|) by {worst:.3e} (max-abs {float(d.max()):.3e})"
    assert float(d.mean()) <= mean_abs, f"{name}: mean-abs {float(d.mean()):.3e} (limit {mean_abs})"
    return float(d.max()), float(d.mean())


def grad_error_report(got, want, max_abs: float = BF16_MAX_ABS) -> dict:
    """How a gradient meets assert_close_grad_bf16's bound: the largest error among elements with |want| <= 2 (where
    the absolute bound alone applies), and how many elements lie beyond `max_abs` and pass on the relative arm."""
    g = got.detach().float().cpu()
    w = want.detach().float().cpu()
    d = (g - w).abs()
    small = w.abs() <= 2.0
    return {"max_abs_where_want_le_2": float(d[small].max()) if small.any() else 0.0,
            "elements": d.numel(), "beyond_abs_bound": int((d > max_abs).sum()),
            "largest_want": float(w.abs().max()), "max_abs": float(d.max()), "mean_abs": float(d.mean())}


def assert_close_lse(got, want, name: str = "lse", max_abs: float = LSE_MAX_ABS):
    g = got.detach().float().cpu()
    w = want.detach().float().cpu()
    inf_g, inf_w = torch.isinf(g), torch.isinf(w)
    assert torch.equal(inf_g, inf_w), f"{name}: infinite entries differ"
    d = (g[~inf_g] - w[~inf_w]).abs()
    mx = float(d.max()) if d.numel() else 0.0
    assert mx <= max_abs, f"{name}: max-abs {mx:.3e} (limit {max_abs})"
    return mx


# ------------------------------------------------------------------ the reference tests' own rule
# test/torch_ops/test_scaled_dot_product_attention.py:165-204: the fused kernel may deviate from
# the high-precision result by at most `fudge` times what the SAME math evaluated in the low
# precision dtype deviates, with per-dtype floors.
_DEFAULT_ATOL = {torch.float16: 1e-3, torch.bfloat16: 1e-3, torch.float32: 1e-5}
_DEFAULT_RTOL = {torch.float16: 1e-3, torch.bfloat16: 1.6e-2, torch.float32: 1.3e-6}


def reference_tolerances(true_value: torch.Tensor, lowp_value: torch.Tensor, fudge: float = 2.0) -> Tuple[float, float]:
    dt = lowp_value.dtype
    dev = true_value.double() - lowp_value.double()
    atol = float(dev.abs().max())
    rel = torch.nan_to_num((dev / true_value.double()).abs(), nan=_DEFAULT_RTOL[dt])
    rtol = float(rel.max())
    atol = fudge * max(atol, _DEFAULT_ATOL[dt])
    rtol = fudge * max(rtol, _DEFAULT_RTOL[dt])
    if rtol > 1e30:
        rtol = _DEFAULT_RTOL[dt]
    return atol, rtol


def assert_close_reference_rule(got, true_value, lowp_value, name: str, fudge: float = 2.0):
    """got: the kernel's result; true_value: fp32/fp64 math; lowp_value: the same math in got's dtype."""
    atol, rtol = reference_tolerances(true_value, lowp_value, fudge)
    g = got.detach().cpu().double()
    t = true_value.double()
    bad = (g - t).abs() > atol + rtol * t.abs()
    assert not bool(bad.any()), (f"{name}: {int(bad.sum())} elements outside atol {atol:.3e} rtol {rtol:.3e} "
                                 f"(max-abs error {float((g - t).abs().max()):.3e})")
    return atol, rtol


# ------------------------------------------------------------------ dropout pattern
def philox4x32_10(counter, key):
    """Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC'11) on
    numpy arrays: counter [..., 4] and key [..., 2] uint32 -> [..., 4] uint32."""
    import numpy as np
    c = [counter[..., i].astype(np.uint64) for i in range(4)]
    k0 = np.uint64(key[0])
    k1 = np.uint64(key[1])
    mask = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0 = np.uint64(0xD2511F53) * c[0]
        p1 = np.uint64(0xCD9E8D57) * c[2]
        hi0, lo0 = p0 >> np.uint64(32), p0 & mask
        hi1, lo1 = p1 >> np.uint64(32), p1 & mask
        c = [hi1 ^ c[1] ^ k0, lo1, hi0 ^ c[3] ^ k1, lo0]
        k0 = (k0 + np.uint64(0x9E3779B9)) & mask
        k1 = (k1 + np.uint64(0xBB67AE85)) & mask
    return np.stack(c, axis=-1).astype(np.uint32)


def dropout_keep_mask(seed: int, offset: int, dropout_p: float, batch: int, heads: int, seqlen_q: int, seqlen_k: int):
    """bool [batch, heads, seqlen_q, seqlen_k], True = kept: the rule of the library's mask kernel restated.
    counter = (key, query // 16, batch*heads_index, offset & 0xffffffff), key = (seed low, seed high ^ offset high); element
    (q, k) is kept when byte (q % 16) of the 16 output bytes is >= round(dropout_p * 256)."""
    import numpy as np
    drop = min(255, max(0, int(dropout_p * 256.0 + 0.5)))
    groups = (seqlen_q + 15) // 16
    bh, g, k = np.meshgrid(np.arange(batch * heads, dtype=np.uint32), np.arange(groups, dtype=np.uint32),
                           np.arange(seqlen_k, dtype=np.uint32), indexing="ij")
    counter = np.stack([k, g, bh, np.full_like(k, offset & 0xFFFFFFFF)], axis=-1)
    out = philox4x32_10(counter, (seed & 0xFFFFFFFF, ((seed >> 32) ^ (offset >> 32)) & 0xFFFFFFFF))   # [BH, G, Lk, 4]
    by = out.view(np.uint8).reshape(batch * heads, groups, seqlen_k, 16)            # little-endian bytes
    keep = by >= drop                                                               # [BH, G, Lk, 16]
    keep = keep.transpose(0, 1, 3, 2).reshape(batch * heads, groups * 16, seqlen_k)[:, :seqlen_q]
    return torch.from_numpy(np.ascontiguousarray(keep)).reshape(batch, heads, seqlen_q, seqlen_k)
