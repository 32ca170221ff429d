"""Generates tests/golden/attention_ref_*.npz by EXECUTING the reference's own test oracle.

The reference (Cambricon/torch_mlu) keeps its parity oracle for this path as two pure-torch
functions inside test/torch_ops/test_scaled_dot_product_attention.py: ``construct_local_mask``
(:46-75) and ``attention_ref`` (:78-161). That file cannot be imported here (it imports
torch_mlu and needs an MLU), so this script parses it, takes exactly those two function
definitions out of the syntax tree and executes them unchanged with torch, einops and math in
scope. Gradients are taken with autograd through ``attention_ref``, as the reference tests do
(:1018-1075). No reference source is copied into this repository - only the numbers it produces.

Run from the repository root, where the reference checkout is available:
    python tests/golden/make_golden.py /path/to/torch_mlu
Inputs are bf16-representable values stored as their bit patterns (uint16); outputs are fp32.
The file also stores ``lse``, which ``attention_ref`` does not return: it is computed here from
the same scaled scores (natural-log logsumexp over visible keys) and is marked derived.
"""
from __future__ import annotations

import ast
import math
import os
import sys

import numpy as np
import torch
from einops import rearrange, repeat

HERE = os.path.dirname(os.path.abspath(__file__))
REL = "test/torch_ops/test_scaled_dot_product_attention.py"

# name, B, Hq, Hkv, Lq, Lk, D, causal, scale
CASES = [
    ("noncausal_d128", 1, 2, 2, 64, 96, 128, False, None),
    ("causal_square_d128", 1, 2, 2, 128, 128, 128, True, None),
    ("causal_lq_lt_lk_d128", 1, 1, 1, 64, 160, 128, True, None),
    ("causal_lq_gt_lk_d128", 1, 1, 1, 160, 96, 128, True, None),
    ("gqa_causal_scale_d128", 1, 4, 2, 96, 96, 128, True, 1.0 / 128),
    ("noncausal_d64_b2", 2, 2, 2, 48, 80, 64, False, None),
]


# Dropout: the reference's device kernel draws the pattern itself, so its tests feed the pattern the operator
# returns back into attention_ref (:1048-1068). Here the pattern comes from this repository's own rule
# (oracle.sdpa_oracle.dropout_keep_mask, a fixed seed / offset pair) and attention_ref is executed with it.
# name, B, Hq, Hkv, Lq, Lk, D, causal, dropout_p, seed, offset
DROPOUT_CASES = [
    ("causal_square_p22", 1, 2, 2, 128, 128, 128, True, 0.22, 20240607, 12),
    ("noncausal_gqa_p48", 2, 4, 2, 96, 160, 64, False, 0.48, 99, (3 << 32) + 5),
]


def load_reference_functions(ref_root: str):
    path = os.path.join(ref_root, REL)
    tree = ast.parse(open(path).read(), filename=path)
    wanted = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in ("construct_local_mask", "attention_ref")]
    assert len(wanted) == 2, "reference test file no longer has the expected functions"
    ns = {"torch": torch, "math": math, "rearrange": rearrange, "repeat": repeat}
    exec(compile(ast.Module(body=wanted, type_ignores=[]), path, "exec"), ns)
    return ns["attention_ref"]


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.view(torch.int16).numpy().view(np.uint16)


def main() -> None:
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <checkout of Cambricon/torch_mlu>")
    ref_root = sys.argv[1]
    attention_ref = load_reference_functions(ref_root)
    for idx, (name, B, Hq, Hkv, Lq, Lk, D, causal, scale) in enumerate(CASES):
        g = torch.Generator().manual_seed(1234 + idx)
        q = torch.randn(B, Hq, Lq, D, generator=g).bfloat16()
        k = torch.randn(B, Hkv, Lk, D, generator=g).bfloat16()
        v = torch.randn(B, Hkv, Lk, D, generator=g).bfloat16()
        dout = torch.randn(B, Hq, Lq, D, generator=g).bfloat16()
        # the reference oracle takes [batch, seq, heads, dim] and returns [batch, heads, seq, dim]
        qf = q.float().transpose(1, 2).detach().requires_grad_(True)
        kf = k.float().transpose(1, 2).detach().requires_grad_(True)
        vf = v.float().transpose(1, 2).detach().requires_grad_(True)
        out, _ = attention_ref(qf, kf, vf, scale=scale, causal=causal, upcast=True)
        out.backward(dout.float())
        dq = qf.grad.transpose(1, 2).contiguous()
        dk = kf.grad.transpose(1, 2).contiguous()
        dv = vf.grad.transpose(1, 2).contiguous()
        # derived (not produced by the reference): logsumexp of the same scaled, masked scores
        sc = (1.0 / math.sqrt(D)) if scale is None else scale
        kk = k.float().repeat_interleave(Hq // Hkv, dim=1)
        scores = torch.einsum("bhtd,bhsd->bhts", q.float() * sc, kk)
        if causal:
            row = torch.arange(Lq).unsqueeze(1)
            col = torch.arange(Lk).unsqueeze(0)
            scores = scores.masked_fill(col > row + Lk - Lq, float("-inf"))
        lse = torch.logsumexp(scores, -1)
        lse = torch.where(torch.isinf(lse), torch.full_like(lse, float("inf")), lse)
        np.savez_compressed(
            os.path.join(HERE, f"attention_ref_{name}.npz"),
            q=bf16_bits(q), k=bf16_bits(k), v=bf16_bits(v), dout=bf16_bits(dout),
            out=out.detach().numpy().astype(np.float32), dq=dq.numpy(), dk=dk.numpy(), dv=dv.numpy(),
            lse_derived=lse.numpy(), causal=np.array(causal), scale=np.array(-1.0 if scale is None else scale),
        )
        print(name, "out", tuple(out.shape), "finite", bool(torch.isfinite(out).all()))
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from oracle.sdpa_oracle import dropout_keep_mask
    for idx, (name, B, Hq, Hkv, Lq, Lk, D, causal, p, seed, offset) in enumerate(DROPOUT_CASES):
        g = torch.Generator().manual_seed(4321 + idx)
        q = torch.randn(B, Hq, Lq, D, generator=g).bfloat16()
        k = torch.randn(B, Hkv, Lk, D, generator=g).bfloat16()
        v = torch.randn(B, Hkv, Lk, D, generator=g).bfloat16()
        dout = torch.randn(B, Hq, Lq, D, generator=g).bfloat16()
        keep = dropout_keep_mask(seed, offset, p, B, Hq, Lq, Lk)
        qf = q.float().transpose(1, 2).detach().requires_grad_(True)
        kf = k.float().transpose(1, 2).detach().requires_grad_(True)
        vf = v.float().transpose(1, 2).detach().requires_grad_(True)
        out, _ = attention_ref(qf, kf, vf, dropout_p=p, dropout_mask=keep, causal=causal, upcast=True)
        out.backward(dout.float())
        np.savez_compressed(
            os.path.join(HERE, f"dropout_ref_{name}.npz"),
            q=bf16_bits(q), k=bf16_bits(k), v=bf16_bits(v), dout=bf16_bits(dout), keep=np.packbits(keep.numpy()),
            keep_shape=np.array(keep.shape), out=out.detach().numpy().astype(np.float32),
            dq=qf.grad.transpose(1, 2).contiguous().numpy(), dk=kf.grad.transpose(1, 2).contiguous().numpy(),
            dv=vf.grad.transpose(1, 2).contiguous().numpy(), causal=np.array(causal), dropout_p=np.array(p),
            seed=np.array(seed, dtype=np.int64), offset=np.array(offset, dtype=np.int64),
        )
        print("dropout", name, "kept", float(keep.float().mean()), "finite", bool(torch.isfinite(out).all()))


if __name__ == "__main__":
    main()
