"""Runs a few launches of one kernel on a sized-down case, for use under a profiler. A profiling harness kept beside
the package because the commands recorded under profiles/ run it; it is not part of the operator interface.

    python -m torch_mlu_b200.profile_case prefill --batch 2 --heads 32 --seqlen 4096 --launches 3
    python -m torch_mlu_b200.profile_case decode  --batch 8 --seqlen-k 32768 --launches 3
    python -m torch_mlu_b200.profile_case backward --batch 2 --heads 16 --seqlen 2048 --launches 3 [--deterministic]
    python -m torch_mlu_b200.profile_case prefill --batch 2 --heads 16 --seqlen 4096 --head-dim 256 --launches 3
    python -m torch_mlu_b200.profile_case helpers  --batch 4 --heads 16 --seqlen 2048 --launches 2

``helpers`` launches the two HBM-bound side kernels: the dropout keep-mask kernel and the bias transpose.

Inputs are device-generated N(0,1) bf16; sizes default to a few hundred MB so that a
multi-pass profiler capture stays short while the working set still exceeds L2.
"""
from __future__ import annotations

import argparse

import torch

from . import dropout, ops


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["prefill", "decode", "backward", "helpers"])
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--heads-kv", type=int, default=0)
    ap.add_argument("--seqlen", type=int, default=4096)
    ap.add_argument("--seqlen-k", type=int, default=32768)
    ap.add_argument("--launches", type=int, default=3)
    ap.add_argument("--non-causal", action="store_true")
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--deterministic", action="store_true", help="backward: the dK/dV + dQ kernels instead of the fused one")
    a = ap.parse_args()
    D = a.head_dim
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0)
    rn = lambda *s: torch.randn(*s, generator=g, device=dev).to(torch.bfloat16)
    hkv = a.heads_kv or a.heads
    if a.kernel == "helpers":
        bias = rn(a.batch, a.heads, a.seqlen, a.seqlen)
        for i in range(a.launches):
            dropout.KeepMasks(1, i, 0.1, a.batch, a.heads, a.seqlen, a.seqlen, dev, not a.non_causal)
            ops._transposed_bias(bias)
    elif a.kernel == "decode":
        hkv = a.heads_kv or 8
        q, k, v = rn(a.batch, a.heads, 1, 128), rn(a.batch, hkv, a.seqlen_k, 128), rn(a.batch, hkv, a.seqlen_k, 128)
        for _ in range(a.launches):
            ops.decode_attention(q, k, v)
    else:
        q, k, v = rn(a.batch, a.heads, a.seqlen, D), rn(a.batch, hkv, a.seqlen, D), rn(a.batch, hkv, a.seqlen, D)
        causal = not a.non_causal
        if a.kernel == "prefill":
            for _ in range(a.launches):
                ops.gqa_prefill(q, k, v, is_causal=causal)
        else:
            do = rn(a.batch, a.heads, a.seqlen, D)
            out, lse = ops.gqa_prefill(q, k, v, is_causal=causal)
            for _ in range(a.launches):
                ops._dense_backward(do, q, k, v, out, lse, causal, D ** -0.5, deterministic=a.deterministic)
    torch.cuda.synchronize()
    print("device status", ops.device_status())


if __name__ == "__main__":
    main()
