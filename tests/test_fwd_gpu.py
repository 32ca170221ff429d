"""GPU parity of the prefill forward kernel against the CPU oracle, through the C ABI.

Tolerances (bf16 outputs vs the fp32 oracle on the same bf16-rounded inputs): max-abs 2e-2,
mean-abs 2e-3; fp32 logsumexp max-abs 1e-5.
"""
import os

import pytest
import torch

from oracle import sdpa_oracle as orc
from test_oracle import GOLDEN, load_golden
from torch_mlu_b200 import _cabi, ops, workloads

pytestmark = pytest.mark.gpu


def run_dense(dev, q, k, v, causal, scale=None):
    out, lse = ops.gqa_prefill(q.to(dev), k.to(dev), v.to(dev), is_causal=causal, scale=scale)
    assert ops.device_status() == 0
    return out, lse


def check_dense(dev, q, k, v, causal, scale=None, oracle=orc.cpu_sdpa_forward):
    out, lse = run_dense(dev, q, k, v, causal, scale)
    o_ref, l_ref = oracle(q, k, v, causal=causal, scale=scale)
    orc.assert_close_bf16(out, o_ref, "out")
    orc.assert_close_lse(lse, l_ref)
    return out, lse


def rand(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g).bfloat16()


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: os.path.basename(p)[14:-4])
def test_forward_matches_reference_golden(cuda_device, native_lib, path):
    g = load_golden(path)
    before = _cabi.launch_count()
    out, lse = run_dense(cuda_device, g["q"], g["k"], g["v"], g["causal"], g["scale"])
    assert _cabi.launch_count() > before
    orc.assert_close_bf16(out, g["out"], "out vs reference attention_ref")
    orc.assert_close_lse(lse, g["lse"])


@pytest.mark.parametrize("B,Hq,Hkv,Lq,Lk,causal", [
    (1, 1, 1, 128, 128, False),
    (2, 4, 4, 512, 512, True),
    (1, 2, 2, 1024, 1024, False),
    (1, 2, 2, 1000, 1000, True),     # ragged tail in both tiles
    (1, 2, 2, 300, 700, True),       # bottom-right causal, Lq < Lk
    (1, 2, 2, 700, 300, True),       # Lq > Lk: leading rows see no key
    (1, 2, 2, 17, 129, False),       # tiny
    (1, 1, 1, 1, 1, True),           # minimum
    (1, 1, 1, 129, 1, False),
    (2, 8, 2, 384, 384, True),       # GQA 4:1
    (1, 8, 1, 256, 512, False),      # MQA
    (1, 2, 2, 257, 255, True),
])
def test_forward_dense_shapes(cuda_device, native_lib, B, Hq, Hkv, Lq, Lk, causal):
    q, k, v = rand((B, Hq, Lq, 128), 1), rand((B, Hkv, Lk, 128), 2), rand((B, Hkv, Lk, 128), 3)
    check_dense(cuda_device, q, k, v, causal)


@pytest.mark.parametrize("B,Hq,Hkv,Lq,Lk,causal", [
    (2, 4, 4, 512, 512, True),
    (1, 8, 2, 300, 700, True),
    (1, 2, 2, 257, 255, False),
    (1, 1, 1, 1, 1, True),
])
def test_forward_head_dim_64(cuda_device, native_lib, B, Hq, Hkv, Lq, Lk, causal):
    g = torch.Generator().manual_seed(4)
    q = torch.randn((B, Hq, Lq, 64), generator=g).bfloat16()
    k = torch.randn((B, Hkv, Lk, 64), generator=g).bfloat16()
    v = torch.randn((B, Hkv, Lk, 64), generator=g).bfloat16()
    check_dense(cuda_device, q, k, v, causal)


def test_config1_on_gpu_with_bf16_rounded_inputs(cuda_device, native_lib):
    """BASELINE config 1 (B2 H8 L256 D64 non-causal, seed 0, scale 1/8) is the reference's own fp32
    CPU case; the GPU path is bf16, so it runs on the bf16-rounded copies of the same inputs and is
    compared with the CPU reference on those copies."""
    c = workloads.config1_cpu_reference()
    q, k, v = c.q.bfloat16(), c.k.bfloat16(), c.v.bfloat16()
    out, lse = check_dense(cuda_device, q, k, v, False, scale=c.softmax_scale)
    assert out.shape == (2, 8, 256, 64) and lse.shape == (2, 8, 256)


def test_forward_scale_and_layouts(cuda_device, native_lib):
    B, H, L, D = 2, 4, 320, 128
    # [B,L,H,D] storage viewed as [B,H,L,D], and a packed QKV buffer sliced into q/k/v
    packed = rand((B, L, 3 * H * D), 5)
    q, k, v = (t.view(B, L, H, D).transpose(1, 2) for t in packed.chunk(3, dim=-1))
    dev = cuda_device
    pk = packed.to(dev)
    qd, kd, vd = (t.view(B, L, H, D).transpose(1, 2) for t in pk.chunk(3, dim=-1))
    for scale in (None, 1.0 / D, 0.3):
        out, lse = ops.gqa_prefill(qd, kd, vd, is_causal=True, scale=scale)
        o_ref, l_ref = orc.cpu_sdpa_forward(q, k, v, causal=True, scale=scale)
        orc.assert_close_bf16(out, o_ref, f"out scale={scale}")
        orc.assert_close_lse(lse, l_ref)


def test_reference_operator_surface(cuda_device, native_lib):
    """_scaled_dot_product_flash_attention returns the reference's 9-tuple (attention.cpp:149-158)."""
    q, k, v = rand((2, 4, 256, 128), 1), rand((2, 4, 256, 128), 2), rand((2, 4, 256, 128), 3)
    dev = cuda_device
    res = ops._scaled_dot_product_flash_attention(q.to(dev), k.to(dev), v.to(dev), 0.0, True, False)
    out, lse, cum_q, cum_k, max_q, max_k, seed, offset, dbg = res
    assert out.shape == q.shape and out.transpose(1, 2).is_contiguous()
    assert lse.shape == (2, 4, 256) and lse.dtype == torch.float32
    assert cum_q.tolist() == [0, 256, 512] and cum_k.dtype == torch.int32
    assert (max_q, max_k) == (256, 256) and dbg.numel() == 0 and seed.numel() == 0
    o_ref, l_ref = orc.cpu_sdpa_forward(q, k, v, causal=True)
    orc.assert_close_bf16(out, o_ref, "out")
    orc.assert_close_lse(lse, l_ref)
    with pytest.raises(RuntimeError, match="same number of heads"):
        ops._scaled_dot_product_flash_attention(q.to(dev), k.to(dev)[:, :2], v.to(dev)[:, :2])


@pytest.mark.parametrize("lens,Hq,Hkv,causal", [
    ([100, 300, 257, 128], 4, 2, True),
    ([512, 64, 1000], 4, 1, False),
    ([1, 2, 3, 255, 256, 257], 2, 2, True),
    ([640], 8, 8, True),
])
def test_forward_varlen(cuda_device, native_lib, lens, Hq, Hkv, causal):
    total = sum(lens)
    q, k, v = rand((total, Hq, 128), 1), rand((total, Hkv, 128), 2), rand((total, Hkv, 128), 3)
    cu = [0]
    for l in lens:
        cu.append(cu[-1] + l)
    dev = cuda_device
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    out, lse, seed, offset, dbg = ops._flash_attention_forward(q.to(dev), k.to(dev), v.to(dev), cu_t, cu_t, max(lens),
                                                               max(lens), 0.0, causal, False)
    assert ops.device_status() == 0
    assert out.shape == q.shape and lse.shape == (Hq, total)
    o_ref, l_ref = orc.varlen_forward(q, k, v, cu, cu, causal=causal)
    orc.assert_close_bf16(out, o_ref, "out")
    orc.assert_close_lse(lse, l_ref)


def test_varlen_different_q_and_k_lengths(cuda_device, native_lib):
    lens_q, lens_k = [64, 200, 31], [128, 200, 400]
    cu_q, cu_k = [0], [0]
    for a, b in zip(lens_q, lens_k):
        cu_q.append(cu_q[-1] + a)
        cu_k.append(cu_k[-1] + b)
    q, k, v = rand((cu_q[-1], 4, 128), 1), rand((cu_k[-1], 2, 128), 2), rand((cu_k[-1], 2, 128), 3)
    dev = cuda_device
    tq = torch.tensor(cu_q, dtype=torch.int32, device=dev)
    tk = torch.tensor(cu_k, dtype=torch.int32, device=dev)
    out, lse, *_ = ops._flash_attention_forward(q.to(dev), k.to(dev), v.to(dev), tq, tk, max(lens_q), max(lens_k), 0.0,
                                                True, False)
    o_ref, l_ref = orc.varlen_forward(q, k, v, cu_q, cu_k, causal=True)
    orc.assert_close_bf16(out, o_ref, "out")
    orc.assert_close_lse(lse, l_ref)


def test_forward_is_deterministic_and_packed_neighbours_do_not_mix(cuda_device, native_lib):
    """Two runs give identical bits, and two packed sequences that share a 128-row tile get their own results
    (writes outside an output are checked in test_guard_bands_gpu.py)."""
    dev = cuda_device
    B, H, L, D = 1, 2, 200, 128
    q, k, v = rand((B, H, L, D), 1).to(dev), rand((B, H, L, D), 2).to(dev), rand((B, H, L, D), 3).to(dev)
    out1, lse1 = ops.gqa_prefill(q, k, v, is_causal=True)
    out2, lse2 = ops.gqa_prefill(q, k, v, is_causal=True)
    assert torch.equal(out1, out2) and torch.equal(lse1, lse2)
    # varlen: the gap rows between two sequences' tiles must not be written by the neighbour
    lens = [130, 70]
    cu = torch.tensor([0, 130, 200], dtype=torch.int32, device=dev)
    qv = rand((200, 2, D), 4).to(dev)
    out, lse, *_ = ops._flash_attention_forward(qv, qv, qv, cu, cu, 130, 130, 0.0, True, False)
    o_ref, l_ref = orc.varlen_forward(qv.cpu(), qv.cpu(), qv.cpu(), [0, 130, 200], [0, 130, 200], causal=True)
    orc.assert_close_bf16(out, o_ref, "out")


def test_config2_shape_on_sampled_heads_and_causality_property(cuda_device, native_lib):
    """Full-size BASELINE config 2 (B4 H32 L4096 D128 causal, seed 1): oracle parity on a
    sample of (batch, head) pairs, plus a size-independent property on the whole tensor:
    perturbing keys/values at positions >= t leaves rows < t bit-identical."""
    dev = cuda_device
    c = workloads.config2_causal_prefill()
    q, k, v = c.q.to(dev), c.k.to(dev), c.v.to(dev)
    out, lse = ops.gqa_prefill(q, k, v, is_causal=True, scale=c.softmax_scale)
    assert ops.device_status() == 0
    for b, h in ((0, 0), (1, 17), (3, 31)):
        o_ref, l_ref = orc.cpu_sdpa_forward(c.q[b:b + 1, h:h + 1], c.k[b:b + 1, h:h + 1], c.v[b:b + 1, h:h + 1],
                                            causal=True, scale=c.softmax_scale)
        orc.assert_close_bf16(out[b:b + 1, h:h + 1], o_ref, f"out[{b},{h}]")
        orc.assert_close_lse(lse[b:b + 1, h:h + 1], l_ref)
    t = 2048 + 77
    k2, v2 = k.clone(), v.clone()
    k2[:, :, t:] = -k2[:, :, t:]
    v2[:, :, t:] = 3.0
    out2, lse2 = ops.gqa_prefill(q, k2, v2, is_causal=True, scale=c.softmax_scale)
    assert torch.equal(out[:, :, :t], out2[:, :, :t]) and torch.equal(lse[:, :, :t], lse2[:, :, :t])
    assert not torch.equal(out[:, :, t:], out2[:, :, t:])
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()


def test_config4_varlen_gqa_scaled_down(cuda_device, native_lib):
    """BASELINE config 4 drawn with the documented recipe at 1/4 of the lengths, every element against the
    oracle (the full-size run is in test_full_size_gpu.py): ragged cu_seqlens, Hq 32 / Hkv 8, causal."""
    dev = cuda_device
    c = workloads.config4_varlen_gqa(num_seqs=8, lo=128, hi=1024)
    cu = c.cu_seqlens.tolist()
    cu_t = c.cu_seqlens.to(dev)
    out, lse, *_ = ops._flash_attention_forward(c.q.to(dev), c.k.to(dev), c.v.to(dev), cu_t, cu_t, max(c.seqlens),
                                                max(c.seqlens), 0.0, True, False, scale=c.softmax_scale)
    o_ref, l_ref = orc.varlen_forward(c.q, c.k, c.v, cu, cu, causal=True, scale=c.softmax_scale)
    orc.assert_close_bf16(out, o_ref, "out")
    orc.assert_close_lse(lse, l_ref)
