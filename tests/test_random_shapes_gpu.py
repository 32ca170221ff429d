"""Seeded random sweep of shapes through forward + backward on the GPU against the CPU oracle.

The fixed-shape tests pin the cases the reference's tests name; this one walks the space between them
(batch, GQA ratio, unequal and ragged lengths around the 128-row tile edges, every head dim, both
dtypes, scale, causal or not, dense and packed varlen) the way the reference's parameter sweeps do
(test/torch_ops/test_scaled_dot_product_attention.py:938-1000). Output and logsumexp keep the fixed tolerances
of the other parity tests. Gradients are held to the reference suite's own rule (:1077-1110: at most 2x, dq 4x,
as far from the fp32 math as the same math run in the 16-bit dtype), because the sweep reaches gradients of
magnitude tens (two keys shared by 500 queries and a GQA group of 4), where an absolute 2e-2 is below one ulp
of the 16-bit result.
"""
import random

import pytest
import torch

from oracle import sdpa_oracle as orc
from torch_mlu_b200 import ops

pytestmark = pytest.mark.gpu

EDGE_LENGTHS = [1, 2, 7, 63, 64, 65, 127, 128, 129, 191, 255, 256, 257, 300, 384, 511, 513, 640]


def draw_case(rng: random.Random):
    hkv = rng.choice([1, 2, 3])
    group = rng.choice([1, 1, 2, 4])
    return dict(B=rng.choice([1, 2, 3]), Hq=hkv * group, Hkv=hkv, Lq=rng.choice(EDGE_LENGTHS), Lk=rng.choice(EDGE_LENGTHS),
                D=rng.choice([64, 128, 128, 128, 32, 96]), causal=rng.random() < 0.6,
                dtype=rng.choice([torch.bfloat16, torch.bfloat16, torch.float16]),
                scale=rng.choice([None, None, 0.05, 0.2]))


def tensors(shape_list, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(s, generator=g).to(dtype) for s in shape_list]


@pytest.mark.parametrize("block", range(12))
def test_dense_random_shapes(cuda_device, native_lib, block):
    dev = cuda_device
    rng = random.Random(1000 + block)
    for i in range(8):
        c = draw_case(rng)
        B, Hq, Hkv, Lq, Lk, D = c["B"], c["Hq"], c["Hkv"], c["Lq"], c["Lk"], c["D"]
        q, k, v, dout = tensors([(B, Hq, Lq, D), (B, Hkv, Lk, D), (B, Hkv, Lk, D), (B, Hq, Lq, D)], 17 * block + i, c["dtype"])
        qd, kd, vd, dd = q.to(dev), k.to(dev), v.to(dev), dout.to(dev)
        out, lse = ops.gqa_prefill(qd, kd, vd, is_causal=c["causal"], scale=c["scale"])
        dq, dk, dv = ops._dense_backward(dd, qd, kd, vd, out, lse, c["causal"], ops.calculate_scale(qd, c["scale"]))
        assert ops.device_status() == 0, c
        o_ref, l_ref = orc.attention_math(q, k, v, causal=c["causal"], scale=c["scale"])
        want = orc.attention_math_backward(q, k, v, dout, causal=c["causal"], scale=c["scale"])
        lowp = orc.attention_math_backward(q, k, v, dout, causal=c["causal"], scale=c["scale"], dtype=c["dtype"])
        tag = f"{c}"
        orc.assert_close_bf16(out, o_ref, "out " + tag)
        orc.assert_close_lse(lse, l_ref, "lse " + tag)
        for name, g, w, lp, fudge in zip(("dq", "dk", "dv"), (dq, dk, dv), want, lowp, (4, 2, 2)):
            orc.assert_close_reference_rule(g, w, lp, name + " " + tag, fudge=fudge)


@pytest.mark.parametrize("block", range(8))
def test_varlen_random_shapes(cuda_device, native_lib, block):
    dev = cuda_device
    rng = random.Random(2000 + block)
    for i in range(4):
        c = draw_case(rng)
        Hq, Hkv, D = c["Hq"], c["Hkv"], c["D"]
        n_seq = rng.choice([1, 2, 5])
        lens_q = [rng.choice(EDGE_LENGTHS) for _ in range(n_seq)]
        same = rng.random() < 0.5
        lens_k = lens_q if same else [rng.choice(EDGE_LENGTHS) for _ in range(n_seq)]
        cu_q, cu_k = [0], [0]
        for a, b in zip(lens_q, lens_k):
            cu_q.append(cu_q[-1] + a)
            cu_k.append(cu_k[-1] + b)
        q, k, v, dout = tensors([(cu_q[-1], Hq, D), (cu_k[-1], Hkv, D), (cu_k[-1], Hkv, D), (cu_q[-1], Hq, D)],
                                31 * block + i, c["dtype"])
        cq = torch.tensor(cu_q, dtype=torch.int32, device=dev)
        ck = torch.tensor(cu_k, dtype=torch.int32, device=dev)
        qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
        out, lse, seed, off, _ = ops._flash_attention_forward(qd, kd, vd, cq, ck, max(lens_q), max(lens_k), 0.0, c["causal"],
                                                              False, scale=c["scale"])
        dq, dk, dv = ops._flash_attention_backward(dout.to(dev), qd, kd, vd, out, lse, cq, ck, max(lens_q), max(lens_k), 0.0,
                                                   c["causal"], seed, off, scale=c["scale"])
        assert ops.device_status() == 0, (c, lens_q, lens_k)
        tag = f"{c} lens_q={lens_q} lens_k={lens_k}"
        # per sequence, with the kernels' bottom-right causal alignment (lengths differ between q and k)
        o_ref, l_ref = orc.varlen_forward(q, k, v, cu_q, cu_k, causal=c["causal"], scale=c["scale"], impl=orc.attention_math)
        orc.assert_close_bf16(out, o_ref, "out " + tag)
        orc.assert_close_lse(lse, l_ref, "lse " + tag)
        def per_sequence_grads(dtype):
            parts = ([], [], [])
            for s in range(n_seq):
                sq, sk = slice(cu_q[s], cu_q[s + 1]), slice(cu_k[s], cu_k[s + 1])
                one = lambda x, sl: x[sl].transpose(0, 1).unsqueeze(0)
                grads = orc.attention_math_backward(one(q, sq), one(k, sk), one(v, sk), one(dout, sq), causal=c["causal"],
                                                    scale=c["scale"], dtype=dtype)
                for dst, g in zip(parts, grads):
                    dst.append(g[0].transpose(0, 1))
            return [torch.cat(x) for x in parts]

        want, lowp = per_sequence_grads(torch.float32), per_sequence_grads(c["dtype"])
        for name, g, w, lp, fudge in zip(("dq", "dk", "dv"), (dq, dk, dv), want, lowp, (4, 2, 2)):
            orc.assert_close_reference_rule(g, w, lp, name + " " + tag, fudge=fudge)
