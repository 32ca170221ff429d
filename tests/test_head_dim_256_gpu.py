"""Head dims above 128 (the reference admits up to 256, sdp_utils.h:231-255, and its value tests run 256:
test/torch_ops/test_scaled_dot_product_attention.py:728-1285): the kernels that keep the stationary operand in
tensor memory, against the CPU oracle through the C ABI.

Tolerances: bf16 / fp16 outputs max-abs 2e-2 and mean-abs 2e-3, fp32 logsumexp 1e-5, gradients max(2e-2, 1e-2 |want|).
"""
import pytest
import torch

from oracle import sdpa_oracle as orc
from torch_mlu_b200 import ops

pytestmark = pytest.mark.gpu


def rand(shape, seed, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g).to(dtype)


@pytest.mark.parametrize("B,Hq,Hkv,Lq,Lk,D,causal", [
    (4, 2, 2, 512, 512, 256, True),      # the reference's own shape (test_...py:728-935), both mask settings
    (4, 2, 2, 512, 512, 256, False),
    (1, 2, 2, 1024, 2048, 256, True),    # from its sweep of lengths: Lq != Lk, bottom-right aligned mask
    (1, 2, 2, 2048, 512, 256, True),     # leading rows see no key
    (1, 1, 1, 128, 64, 256, False),      # one block
    (1, 1, 1, 1, 1, 256, True),          # minimum
    (2, 4, 2, 333, 777, 256, True),      # ragged lengths, GQA 2:1
    (1, 8, 1, 200, 130, 192, False),     # head_dim 192 (MQA): the last 64 columns are padding
    (2, 2, 2, 257, 255, 136, True),      # head_dim 136: padding inside a 64-column box
    (1, 2, 2, 130, 4100, 160, False),    # more blocks than ring slots several times over
])
def test_forward_head_dims_above_128(cuda_device, native_lib, B, Hq, Hkv, Lq, Lk, D, causal):
    dev = cuda_device
    q, k, v = rand((B, Hq, Lq, D), 1), rand((B, Hkv, Lk, D), 2), rand((B, Hkv, Lk, D), 3)
    out, lse = ops.gqa_prefill(q.to(dev), k.to(dev), v.to(dev), is_causal=causal)
    assert ops.device_status() == 0
    o_ref, l_ref = orc.cpu_sdpa_forward(q, k, v, causal=causal)
    orc.assert_close_bf16(out, o_ref, "out")
    orc.assert_close_lse(lse, l_ref)


def test_forward_head_dim_256_fp16_scale_and_layout(cuda_device, native_lib):
    dev = cuda_device
    B, H, L, D = 2, 3, 320, 256
    packed = rand((B, L, 3 * H * D), 5, torch.float16)
    q, k, v = (t.view(B, L, H, D).transpose(1, 2) for t in packed.chunk(3, dim=-1))
    qd, kd, vd = (t.view(B, L, H, D).transpose(1, 2) for t in packed.to(dev).chunk(3, dim=-1))
    for scale in (None, 0.01):
        out, lse = ops.gqa_prefill(qd, kd, vd, is_causal=True, scale=scale)
        o_ref, l_ref = orc.cpu_sdpa_forward(q, k, v, causal=True, scale=scale)
        orc.assert_close_bf16(out, o_ref, f"out scale={scale}")
        orc.assert_close_lse(lse, l_ref)


@pytest.mark.parametrize("lens,Hq,Hkv,D,causal", [
    ([100, 300, 257, 128], 4, 2, 256, True),
    ([1, 2, 255, 64, 65], 2, 2, 256, False),
    ([640, 130], 4, 1, 192, True),
])
def test_forward_packed_head_dims_above_128(cuda_device, native_lib, lens, Hq, Hkv, D, causal):
    dev = cuda_device
    total = sum(lens)
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    q, k, v = rand((total, Hq, D), 1), rand((total, Hkv, D), 2), rand((total, Hkv, D), 3)
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    out, lse, *_ = ops._flash_attention_forward(q.to(dev), k.to(dev), v.to(dev), cu_t, cu_t, max(lens), max(lens), 0.0, causal, False)
    assert ops.device_status() == 0
    o_ref, l_ref = orc.varlen_forward(q, k, v, cu, cu, causal=causal)
    orc.assert_close_bf16(out, o_ref, "out")
    orc.assert_close_lse(lse, l_ref)
