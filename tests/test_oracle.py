"""CPU checks of the oracle itself: against the golden vectors produced by the reference's
attention_ref, between its independent statements, and on the reference's CPU-runnable config."""
import glob
import math
import os

import numpy as np
import pytest
import torch

from oracle import c_oracle
from oracle import sdpa_oracle as orc
from torch_mlu_b200 import workloads

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "attention_ref_*.npz")))


def load_golden(path):
    z = np.load(path)
    bits = lambda a: torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
    scale = float(z["scale"])
    return dict(q=bits(z["q"]), k=bits(z["k"]), v=bits(z["v"]), dout=bits(z["dout"]),
                out=torch.from_numpy(z["out"]), dq=torch.from_numpy(z["dq"]), dk=torch.from_numpy(z["dk"]),
                dv=torch.from_numpy(z["dv"]), lse=torch.from_numpy(z["lse_derived"]),
                causal=bool(z["causal"]), scale=None if scale < 0 else scale)


def test_golden_files_present():
    assert len(GOLDEN) >= 6


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[14:-4] for p in GOLDEN])
def test_oracle_statements_match_reference_golden(path):
    g = load_golden(path)
    kw = dict(causal=g["causal"], scale=g["scale"])
    # explicit math (fp32): same formulation as the reference oracle -> tight
    out, lse = orc.attention_math(g["q"], g["k"], g["v"], **kw)
    assert orc.error_stats(out, g["out"])[0] < 2e-5
    orc.assert_close_lse(lse, g["lse"], max_abs=5e-6)
    dq, dk, dv = orc.attention_math_backward(g["q"], g["k"], g["v"], g["dout"], **kw)
    for name, got in (("dq", dq), ("dk", dk), ("dv", dv)):
        assert orc.error_stats(got, g[name])[0] < 1e-4, name
    # torch CPU fused SDPA (fp32)
    out2, lse2 = orc.cpu_sdpa_forward(g["q"], g["k"], g["v"], **kw)
    assert orc.error_stats(out2, g["out"])[0] < 2e-5
    orc.assert_close_lse(lse2, g["lse"], max_abs=5e-6)
    dq2, dk2, dv2 = orc.cpu_sdpa_backward(g["dout"], g["q"], g["k"], g["v"], out2, lse2, **kw)
    for name, got in (("dq", dq2), ("dk", dk2), ("dv", dv2)):
        assert orc.error_stats(got, g[name])[0] < 1e-4, name
    # plain C, fp64 accumulation
    out3, lse3 = c_oracle.forward(g["q"], g["k"], g["v"], **kw)
    assert orc.error_stats(out3, g["out"])[0] < 2e-5
    orc.assert_close_lse(lse3, g["lse"], max_abs=5e-6)
    dq3, dk3, dv3 = c_oracle.backward(g["q"], g["k"], g["v"], g["dout"], **kw)
    for name, got in (("dq", dq3), ("dk", dk3), ("dv", dv3)):
        assert orc.error_stats(got, g[name])[0] < 1e-4, name


def test_config1_cpu_reference_case():
    """BASELINE config 1: fp32 B2 H8 L256 D64 non-causal, seed 0 - the case the reference path
    (torch CPU SDPA) runs as is. LSE is the natural-log logsumexp of the scaled scores."""
    c = workloads.config1_cpu_reference()
    out, lse = orc.cpu_sdpa_forward(c.q, c.k, c.v, causal=False, scale=c.softmax_scale)
    out_m, lse_m = orc.attention_math(c.q, c.k, c.v, causal=False, scale=c.softmax_scale, dtype=torch.float64)
    assert orc.error_stats(out, out_m)[0] < 5e-6
    assert orc.error_stats(lse, lse_m)[0] < 5e-6
    scores = torch.einsum("bhtd,bhsd->bhts", c.q.double(), c.k.double()) / math.sqrt(64)
    assert orc.error_stats(lse, torch.logsumexp(scores, -1))[0] < 5e-6
    assert c.forward_flops() == pytest.approx(2.684e8, rel=1e-3)


def test_config4_lengths_are_the_documented_draw():
    g = torch.Generator().manual_seed(3)
    lens = torch.randint(512, 4097, (16,), generator=g).tolist()
    assert lens == workloads.CONFIG4_SEQLENS
    assert sum(lens) == 34004 and max(lens) == 4038


def test_varlen_oracle_equals_per_sequence_dense():
    g = torch.Generator().manual_seed(7)
    lens = [5, 33, 1, 64]
    cu = [0]
    for l in lens:
        cu.append(cu[-1] + l)
    q = torch.randn(cu[-1], 4, 32, generator=g)
    k = torch.randn(cu[-1], 2, 32, generator=g)
    v = torch.randn(cu[-1], 2, 32, generator=g)
    out, lse = orc.varlen_forward(q, k, v, cu, cu, causal=True)
    assert out.shape == q.shape and lse.shape == (4, cu[-1])
    i = 1
    o1, l1 = orc.attention_math(q[cu[i]:cu[i + 1]].transpose(0, 1)[None], k[cu[i]:cu[i + 1]].transpose(0, 1)[None],
                                v[cu[i]:cu[i + 1]].transpose(0, 1)[None], causal=True)
    assert orc.error_stats(out[cu[i]:cu[i + 1]], o1[0].transpose(0, 1))[0] < 1e-5
    assert orc.error_stats(lse[:, cu[i]:cu[i + 1]], l1[0])[0] < 1e-5
    dout = torch.randn(q.shape, generator=g)
    dq, dk, dv = orc.varlen_backward(dout, q, k, v, cu, cu, causal=True)
    assert dq.shape == q.shape and dk.shape == k.shape and dv.shape == v.shape


def test_fully_masked_rows_follow_library_convention():
    """Lq > Lk with bottom-right causal: the first Lq-Lk rows see no key -> out 0, lse +inf."""
    g = torch.Generator().manual_seed(11)
    q = torch.randn(1, 1, 6, 16, generator=g)
    k = torch.randn(1, 1, 4, 16, generator=g)
    v = torch.randn(1, 1, 4, 16, generator=g)
    for fn in (orc.attention_math, orc.cpu_sdpa_forward, c_oracle.forward):
        out, lse = fn(q, k, v, causal=True)
        assert torch.all(out[0, 0, :2] == 0) and torch.all(torch.isinf(lse[0, 0, :2]) & (lse[0, 0, :2] > 0))
        assert torch.isfinite(lse[0, 0, 2:]).all()


def test_reference_tolerance_rule_floors_and_fudge():
    """reference_tolerances restates get_tolerances
    (test/torch_ops/test_scaled_dot_product_attention.py:188-204)."""
    true = torch.tensor([1.0, 2.0, 4.0])
    lowp = torch.tensor([1.0, 2.0, 4.0]).bfloat16()
    atol, rtol = orc.reference_tolerances(true, lowp)          # no deviation: the per-dtype floors x 2
    assert atol == pytest.approx(2e-3) and rtol == pytest.approx(3.2e-2)
    lowp = torch.tensor([1.0, 2.0, 4.5]).bfloat16()
    atol, rtol = orc.reference_tolerances(true, lowp, fudge=4)
    assert atol == pytest.approx(4 * 0.5) and rtol == pytest.approx(4 * 0.125)
    orc.assert_close_reference_rule(torch.tensor([1.0, 2.0, 5.0]), true, lowp, "x", fudge=4)
    with pytest.raises(AssertionError):
        orc.assert_close_reference_rule(torch.tensor([1.0, 2.0, 9.0]), true, lowp, "x")


def test_philox4x32_10_known_answers():
    """The dropout pattern's generator against the published known-answer vectors of Philox4x32-10 (the three
    philox4x32 10-round lines of the Random123 distribution's kat_vectors: zero, all-ones and pi-digit inputs)."""
    import numpy as np
    cases = [
        ((0, 0, 0, 0), (0, 0), (0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8)),
        ((0xFFFFFFFF,) * 4, (0xFFFFFFFF, 0xFFFFFFFF), (0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD)),
        ((0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344), (0xA4093822, 0x299F31D0),
         (0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1)),
    ]
    for counter, key, want in cases:
        got = orc.philox4x32_10(np.array([counter], dtype=np.uint32), key)[0]
        assert tuple(int(x) for x in got) == want


def test_dropout_keep_mask_rule():
    """Keep rate, dependence on seed / offset / head, and the byte rule: with p = 0.5 an element is kept exactly
    when its byte is >= 128."""
    a = orc.dropout_keep_mask(7, 0, 0.25, 2, 3, 200, 300)
    assert a.shape == (2, 3, 200, 300) and abs(float(a.float().mean()) - 0.75) < 5e-3
    assert not torch.equal(a, orc.dropout_keep_mask(7, 1, 0.25, 2, 3, 200, 300))
    assert not torch.equal(a, orc.dropout_keep_mask(8, 0, 0.25, 2, 3, 200, 300))
    assert not torch.equal(a[0, 0], a[0, 1]) and not torch.equal(a[0, 0], a[1, 0])
    # a longer sequence extends the pattern, it does not change it
    assert torch.equal(a[..., :100, :150], orc.dropout_keep_mask(7, 0, 0.25, 2, 3, 100, 150))


DROPOUT_GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "dropout_ref_*.npz")))


def load_dropout_golden(path):
    z = np.load(path)
    bits = lambda a: torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
    shape = tuple(int(x) for x in z["keep_shape"])
    keep = torch.from_numpy(np.unpackbits(z["keep"])[:int(np.prod(shape))].astype(bool)).reshape(shape)
    return dict(q=bits(z["q"]), k=bits(z["k"]), v=bits(z["v"]), dout=bits(z["dout"]), keep=keep,
                out=torch.from_numpy(z["out"]), dq=torch.from_numpy(z["dq"]), dk=torch.from_numpy(z["dk"]),
                dv=torch.from_numpy(z["dv"]), causal=bool(z["causal"]), p=float(z["dropout_p"]), seed=int(z["seed"]),
                offset=int(z["offset"]))


@pytest.mark.parametrize("path", DROPOUT_GOLDEN, ids=[os.path.basename(p)[12:-4] for p in DROPOUT_GOLDEN])
def test_oracle_with_dropout_matches_reference_golden(path):
    """attention_math with a keep-mask against the reference's attention_ref executed with the same mask
    (tests/golden/make_golden.py); the stored mask is what the pattern rule gives for the stored seed / offset."""
    g = load_dropout_golden(path)
    B, H, Lq, Lk = g["keep"].shape
    assert torch.equal(g["keep"], orc.dropout_keep_mask(g["seed"], g["offset"], g["p"], B, H, Lq, Lk))
    kw = dict(causal=g["causal"], keep=g["keep"], dropout_p=g["p"])
    out, _ = orc.attention_math(g["q"], g["k"], g["v"], **kw)
    assert orc.error_stats(out, g["out"])[0] < 2e-5
    for name, got in zip(("dq", "dk", "dv"), orc.attention_math_backward(g["q"], g["k"], g["v"], g["dout"], **kw)):
        assert orc.error_stats(got, g[name])[0] < 1e-4, name
