"""Scaled-dot-product-attention backend toggles, mirroring ``torch.backends.mlu`` of the
reference (torch_mlu/backends/mlu/__init__.py:106-188): the same names forward to torch's
global SDP flags, which is what decides whether ``F.scaled_dot_product_attention`` reaches the
flash operators this package implements."""
from __future__ import annotations

import contextlib
from enum import IntEnum

import torch


class SDPBackend(IntEnum):
    """Same values as the reference enum (backends/mlu/__init__.py:106-118, sdp_utils.h:16-21)."""
    ERROR = -1
    MATH = 0
    FLASH_ATTENTION = 1
    EFFICIENT_ATTENTION = 2


def flash_sdp_enabled() -> bool:
    return torch._C._get_flash_sdp_enabled()


def enable_flash_sdp(enabled: bool) -> None:
    torch._C._set_sdp_use_flash(enabled)


def mem_efficient_sdp_enabled() -> bool:
    return torch._C._get_mem_efficient_sdp_enabled()


def enable_mem_efficient_sdp(enabled: bool) -> None:
    torch._C._set_sdp_use_mem_efficient(enabled)


def math_sdp_enabled() -> bool:
    return torch._C._get_math_sdp_enabled()


def enable_math_sdp(enabled: bool) -> None:
    torch._C._set_sdp_use_math(enabled)


def cudnn_sdp_enabled() -> bool:
    """The installed torch has a fourth backend (cuDNN attention) the reference's torch 2.1 does
    not know; on sm_100 torch prefers it over flash."""
    getter = getattr(torch._C, "_get_cudnn_sdp_enabled", None)
    return bool(getter()) if getter else False


def enable_cudnn_sdp(enabled: bool) -> None:
    setter = getattr(torch._C, "_set_sdp_use_cudnn", None)
    if setter:
        setter(enabled)


@contextlib.contextmanager
def sdp_kernel(enable_flash: bool = True, enable_math: bool = True, enable_mem_efficient: bool = True,
               enable_cudnn=None):
    """Temporarily enable/disable the SDPA backends; previous flags are restored on exit.

    Same three flags as the reference. The cuDNN backend, unknown to the reference, follows its
    intent: it stays on only when no backend was switched off (or when ``enable_cudnn`` says so),
    so ``sdp_kernel(enable_flash=True, enable_math=False, enable_mem_efficient=False)`` really
    means "flash only"."""
    if enable_cudnn is None:
        enable_cudnn = enable_flash and enable_math and enable_mem_efficient and cudnn_sdp_enabled()
    previous = (flash_sdp_enabled(), mem_efficient_sdp_enabled(), math_sdp_enabled(), cudnn_sdp_enabled())
    try:
        enable_flash_sdp(enable_flash)
        enable_mem_efficient_sdp(enable_mem_efficient)
        enable_math_sdp(enable_math)
        enable_cudnn_sdp(enable_cudnn)
        yield {}
    finally:
        enable_flash_sdp(previous[0])
        enable_mem_efficient_sdp(previous[1])
        enable_math_sdp(previous[2])
        enable_cudnn_sdp(previous[3])
