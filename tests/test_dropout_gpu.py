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
    m = dropout.KeepMasks(0x1234567890ABCDEF, 77, p, B, H, Lq, Lk, cuda_device)
    want = orc.dropout_keep_mask(0x1234567890ABCDEF, 77, p, B, H, Lq, Lk)
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
