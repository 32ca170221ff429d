"""torch_mlu_b200: a B200 (sm_100a) drop-in for torch_mlu's attention hot path.

Scaled-dot-product attention forward/backward and split-KV decode, behind the reference's
operator names (see ``ops``), over a plain C ABI (``include/sdpa_b200.h``) into hand-written
CUDA. Importing the package does not need a GPU; calling an op does.
"""
from . import _cabi  # noqa: F401
from .ops import (  # noqa: F401
    _flash_attention_backward,
    _flash_attention_forward,
    _scaled_dot_product_flash_attention,
    _scaled_dot_product_flash_attention_backward,
    calculate_scale,
    decode_attention,
    gqa_prefill,
)

__version__ = "0.1.0"
