"""GPU parity of the split-KV decode kernel against the CPU oracle, through the C ABI."""
import pytest
import torch

from oracle import sdpa_oracle as orc
from torch_mlu_b200 import ops, workloads

pytestmark = pytest.mark.gpu


def rand(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g).bfloat16()


@pytest.mark.parametrize("B,Hq,Hkv,Lk,splits", [
    (2, 8, 2, 1000, 1),
    (2, 8, 2, 1000, 4),
    (1, 4, 4, 4096, 0),
    (2, 32, 2, 777, 3),     # 16 query heads per KV head: both fragment row halves
    (1, 40, 1, 2048, 2),    # 40:1 MQA, three head chunks
    (3, 8, 8, 1, 1),        # single key
    (1, 8, 2, 63, 5),       # more splits than 64-key steps: empty splits
    (1, 32, 8, 8192, 0),
])
def test_decode_matches_oracle(cuda_device, native_lib, B, Hq, Hkv, Lk, splits):
    q, k, v = rand((B, Hq, 1, 128), 1), rand((B, Hkv, Lk, 128), 2), rand((B, Hkv, Lk, 128), 3)
    dev = cuda_device
    out, lse = ops.decode_attention(q.to(dev), k.to(dev), v.to(dev), num_splits=splits)
    o_ref, l_ref = orc.cpu_sdpa_forward(q, k, v, causal=False)
    orc.assert_close_bf16(out, o_ref, "out")
    orc.assert_close_lse(lse, l_ref)


@pytest.mark.parametrize("B,Hq,Hkv,Lk,splits", [(2, 8, 2, 1000, 4), (1, 32, 2, 777, 3), (1, 4, 4, 4096, 0)])
def test_decode_head_dim_64(cuda_device, native_lib, B, Hq, Hkv, Lk, splits):
    g = torch.Generator().manual_seed(8)
    q = torch.randn((B, Hq, 1, 64), generator=g).bfloat16()
    k = torch.randn((B, Hkv, Lk, 64), generator=g).bfloat16()
    v = torch.randn((B, Hkv, Lk, 64), generator=g).bfloat16()
    dev = cuda_device
    out, lse = ops.decode_attention(q.to(dev), k.to(dev), v.to(dev), num_splits=splits)
    o_ref, l_ref = orc.cpu_sdpa_forward(q, k, v, causal=False)
    orc.assert_close_bf16(out, o_ref, "out")
    orc.assert_close_lse(lse, l_ref)


def test_decode_auto_dispatch_and_strided_cache(cuda_device, native_lib):
    """Lq == 1 reaches the decode kernel through the dense op too; the cache may be a
    [B, L, H, D] buffer viewed as [B, H, L, D]."""
    dev = cuda_device
    B, Hq, Hkv, Lk = 2, 8, 2, 1500
    q = rand((B, Hq, 1, 128), 1)
    kc = rand((B, Lk, Hkv, 128), 2).transpose(1, 2)
    vc = rand((B, Lk, Hkv, 128), 3).transpose(1, 2)
    out, lse = ops.decode_attention(q.to(dev), kc.to(dev), vc.to(dev))
    o_ref, l_ref = orc.cpu_sdpa_forward(q, kc, vc)
    orc.assert_close_bf16(out, o_ref, "out")
    orc.assert_close_lse(lse, l_ref)
    qq = rand((B, 4, 1, 128), 4)
    kk = rand((B, 4, 300, 128), 5)
    res = ops._scaled_dot_product_flash_attention(qq.to(dev), kk.to(dev), kk.to(dev))
    o_ref, l_ref = orc.cpu_sdpa_forward(qq, kk, kk)
    orc.assert_close_bf16(res[0], o_ref, "out")
    orc.assert_close_lse(res[1][..., :1], l_ref)  # the operator pads the logsumexp to 16 rows


def test_decode_split_count_does_not_change_the_answer_much(cuda_device, native_lib):
    """Size-independent property at the benchmark's KV length: any split count gives the same
    result up to fp32 merge rounding, and equals the oracle on a sampled batch element."""
    dev = cuda_device
    c = workloads.config5_decode(batch=4, seqlen_k=32768)
    q, k, v = c.q.to(dev), c.k.to(dev), c.v.to(dev)
    base_o, base_l = ops.decode_attention(q, k, v, scale=c.softmax_scale, num_splits=1)
    for s in (0, 7, 16, 64):
        o, l = ops.decode_attention(q, k, v, scale=c.softmax_scale, num_splits=s)
        assert orc.error_stats(o, base_o)[0] <= 2e-3
        assert orc.error_stats(l, base_l)[0] <= 2e-6
    o_ref, l_ref = orc.cpu_sdpa_forward(c.q[1:2], c.k[1:2], c.v[1:2], scale=c.softmax_scale)
    orc.assert_close_bf16(base_o[1:2], o_ref, "out")
    orc.assert_close_lse(base_l[1:2], l_ref)
