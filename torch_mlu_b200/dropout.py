"""Dropout keep-masks for the attention operators (the C ABI's sdpa_b200_dropout_keep_mask).

The reference returns a Philox (seed, offset) pair from its forward operators and replays it in the
backward ones (FlashAttention_internal.cpp:190-214, 46-49). Here the pair selects a bit pattern that a small
kernel writes once per call in two orientations; the attention kernels only read bits.
"""
from __future__ import annotations

from typing import Tuple

import torch

from . import _cabi


def padded(length: int) -> int:
    return (length + 127) // 128 * 128


class KeepMasks:
    """keep_rows [B*H, Lq_pad, Lk_pad/32] and keep_cols [B*H, Lk_pad, Lq_pad/32] int32 words on the device."""

    def __init__(self, seed: int, offset: int, dropout_p: float, batch: int, heads: int, seqlen_q: int, seqlen_k: int,
                 device: torch.device, is_causal: bool = False):
        if not (0.0 < dropout_p < 1.0):
            raise ValueError(f"dropout_p must be inside (0, 1), got {dropout_p}")
        self.shape = (batch, heads, seqlen_q, seqlen_k)
        self.dropout_p = float(dropout_p)
        self.seed, self.offset = int(seed), int(offset)
        lq, lk = padded(seqlen_q), padded(seqlen_k)
        self.rows = torch.empty((batch * heads, lq, lk // 32), dtype=torch.int32, device=device)
        self.cols = torch.empty((batch * heads, lk, lq // 32), dtype=torch.int32, device=device)
        lib = _cabi.load()
        with torch.cuda.device(device):
            stream = torch.cuda.current_stream(device).cuda_stream
            _cabi.check(lib.sdpa_b200_dropout_keep_mask(self.seed & (2 ** 64 - 1), self.offset & (2 ** 64 - 1), self.dropout_p,
                                                        batch, heads, seqlen_q, seqlen_k, int(bool(is_causal)),
                                                        self.rows.data_ptr(), self.cols.data_ptr(), stream),
                        "sdpa_b200_dropout_keep_mask")

    def dense(self) -> torch.Tensor:
        """bool [B, H, Lq, Lk], True = kept (what the reference's debug mask encodes as > 0)."""
        B, H, Lq, Lk = self.shape
        bits = (self.rows.unsqueeze(-1) >> torch.arange(32, device=self.rows.device, dtype=torch.int32)) & 1
        return bits.reshape(B * H, self.rows.size(1), -1)[:, :Lq, :Lk].reshape(B, H, Lq, Lk).bool()

    def dense_from_cols(self) -> torch.Tensor:
        B, H, Lq, Lk = self.shape
        bits = (self.cols.unsqueeze(-1) >> torch.arange(32, device=self.cols.device, dtype=torch.int32)) & 1
        return bits.reshape(B * H, self.cols.size(1), -1)[:, :Lk, :Lq].transpose(1, 2).reshape(B, H, Lq, Lk).bool()


class KeepMasksVarlen:
    """The packed form: keep_rows [H, total_q + 128, Lk_pad/32] and keep_cols [H, total_k + 128, Lq_pad/32], rows
    addressed by packed token index, bits by the position inside the token's sequence. Sequence b gets the bits
    batch index b would get in the dense form."""

    def __init__(self, seed: int, offset: int, dropout_p: float, heads: int, cu_q: torch.Tensor, cu_k: torch.Tensor,
                 total_q: int, total_k: int, max_q: int, max_k: int, is_causal: bool = False):
        if not (0.0 < dropout_p < 1.0):
            raise ValueError(f"dropout_p must be inside (0, 1), got {dropout_p}")
        device = cu_q.device
        self.dropout_p = float(dropout_p)
        self.seed, self.offset = int(seed), int(offset)
        self.heads, self.max_q, self.max_k = heads, max_q, max_k
        self.cu_q, self.cu_k = cu_q, cu_k
        self.rows = torch.zeros((heads, total_q + 128, padded(max_k) // 32), dtype=torch.int32, device=device)
        self.cols = torch.zeros((heads, total_k + 128, padded(max_q) // 32), dtype=torch.int32, device=device)
        lib = _cabi.load()
        with torch.cuda.device(device):
            stream = torch.cuda.current_stream(device).cuda_stream
            _cabi.check(lib.sdpa_b200_dropout_keep_mask_varlen(
                self.seed & (2 ** 64 - 1), self.offset & (2 ** 64 - 1), self.dropout_p, cu_q.numel() - 1, heads,
                cu_q.data_ptr(), cu_k.data_ptr(), total_q, total_k, max_q, max_k, int(bool(is_causal)), self.rows.data_ptr(),
                self.cols.data_ptr(), stream), "sdpa_b200_dropout_keep_mask_varlen")

    def dense(self) -> torch.Tensor:
        """bool [B, H, max_q, max_k], True = kept, False outside a sequence (reads cu_seqlens back to the host)."""
        cu_q, cu_k = self.cu_q.tolist(), self.cu_k.tolist()
        out = torch.zeros((len(cu_q) - 1, self.heads, self.max_q, self.max_k), dtype=torch.bool, device=self.rows.device)
        shifts = torch.arange(32, device=self.rows.device, dtype=torch.int32)
        for b in range(len(cu_q) - 1):
            lq, lk = cu_q[b + 1] - cu_q[b], cu_k[b + 1] - cu_k[b]
            words = self.rows[:, cu_q[b]:cu_q[b + 1]]
            bits = ((words.unsqueeze(-1) >> shifts) & 1).reshape(self.heads, lq, -1)[:, :, :lk]
            out[b, :, :lq, :lk] = bits.bool()
        return out


class _LastForward:
    """The keep-masks of the most recent forward call per device. A backward operator that is handed the same Philox
    pair for the same shapes takes them from here instead of drawing the whole pattern a second time (it is the
    same pattern by construction); anything else is drawn afresh. One entry per device: one forward, one backward."""

    _slots: dict = {}

    @classmethod
    def put(cls, device: torch.device, key: tuple, masks) -> None:
        cls._slots[device.index] = (key, masks)

    @classmethod
    def take(cls, device: torch.device, key: tuple):
        slot = cls._slots.get(device.index)
        if slot is None or slot[0] != key:
            return None
        del cls._slots[device.index]
        return slot[1]


def dense_masks(seed: int, offset: int, dropout_p: float, batch: int, heads: int, seqlen_q: int, seqlen_k: int,
                device: torch.device, is_causal: bool, *, forward: bool) -> KeepMasks:
    """KeepMasks for one dense operator call: a forward call draws them and leaves them for its backward, a backward
    call takes what its forward left or draws them again from the pair."""
    key = ("dense", int(seed), int(offset), float(dropout_p), batch, heads, seqlen_q, seqlen_k, bool(is_causal))
    if not forward:
        hit = _LastForward.take(device, key)
        if hit is not None:
            return hit
    masks = KeepMasks(seed, offset, dropout_p, batch, heads, seqlen_q, seqlen_k, device, is_causal)
    if forward:
        _LastForward.put(device, key, masks)
    return masks


def packed_masks(seed: int, offset: int, dropout_p: float, heads: int, cu_q: torch.Tensor, cu_k: torch.Tensor, total_q: int,
                 total_k: int, max_q: int, max_k: int, is_causal: bool, *, forward: bool) -> KeepMasksVarlen:
    """The same for packed (varlen) calls; the offsets tensors are part of the key by identity of their memory."""
    key = ("packed", int(seed), int(offset), float(dropout_p), heads, cu_q.data_ptr(), cu_k.data_ptr(), total_q, total_k, max_q,
           max_k, bool(is_causal))
    if not forward:
        hit = _LastForward.take(cu_q.device, key)
        if hit is not None:
            return hit
    masks = KeepMasksVarlen(seed, offset, dropout_p, heads, cu_q, cu_k, total_q, total_k, max_q, max_k, is_causal)
    if forward:
        _LastForward.put(cu_q.device, key, masks)
    return masks


def draw_seed_and_offset(device: torch.device, elements: int) -> Tuple[int, int]:
    """(seed, offset) for one call from the device's default generator, which moves on by the number of Philox
    calls the elements stand for (what getCounterOffset does, FlashAttention_internal.cpp:46-49): the same
    stream every other torch consumer draws from, so torch.cuda.manual_seed makes a run repeatable."""
    gen = torch.cuda.default_generators[device.index if device.index is not None else torch.cuda.current_device()]
    seed, offset = gen.initial_seed(), gen.get_offset()
    gen.set_offset(offset + ((elements + 3) // 4 + 3) // 4 * 4)  # the generator keeps offsets in multiples of 4
    return seed, offset
