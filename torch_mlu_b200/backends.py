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


@contextlib.contextmanager
def sdp_kernel(enable_flash: bool = True, enable_math: bool = True, enable_mem_efficient: bool = True):
    """Temporarily enable/disable the three SDPA backends; previous flags are restored on exit."""
    previous = (flash_sdp_enabled(), mem_efficient_sdp_enabled(), math_sdp_enabled())
    try:
        enable_flash_sdp(enable_flash)
        enable_mem_efficient_sdp(enable_mem_efficient)
        enable_math_sdp(enable_math)
        yield {}
    finally:
        enable_flash_sdp(previous[0])
        enable_mem_efficient_sdp(previous[1])
        enable_math_sdp(previous[2])
