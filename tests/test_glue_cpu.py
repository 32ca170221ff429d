"""The dispatcher glue without a GPU: it builds, loads, defines the four operators with the
reference's schemas and the backend toggles behave like the reference's."""
import re

import torch

from torch_mlu_b200 import backends, torch_glue

# codegen/mlu_functions.yaml:1313-1316 of the reference
REFERENCE_SCHEMAS = {
    "_scaled_dot_product_flash_attention": "(Tensor query, Tensor key, Tensor value, float dropout_p=0.0, bool is_causal=False, bool return_debug_mask=False, *, float? scale=None) -> (Tensor ouput, Tensor logsumexp, Tensor cum_seq_q, Tensor cum_seq_k, int max_q, int max_k, Tensor philox_seed, Tensor philox_offset, Tensor debug_attn_mask)",
    "_scaled_dot_product_flash_attention_backward": "(Tensor grad_out, Tensor query, Tensor key, Tensor value, Tensor out, Tensor logsumexp, Tensor cum_seq_q, Tensor cum_seq_k, int max_q, int max_k, float dropout_p, bool is_causal, Tensor philox_seed, Tensor philox_offset, *, float? scale=None) -> (Tensor grad_query, Tensor grad_key, Tensor grad_value)",
    "_flash_attention_forward": "(Tensor query, Tensor key, Tensor value, Tensor cum_seq_q, Tensor cum_seq_k, int max_q, int max_k, float dropout_p, bool is_causal, bool return_debug_mask, *, float? scale=None) -> (Tensor output, Tensor softmax_logsumexp, Tensor philox_seed, Tensor philox_offset, Tensor debug_attn_mask)",
    "_flash_attention_backward": "(Tensor grad_out, Tensor query, Tensor key, Tensor value, Tensor out, Tensor logsumexp, Tensor cum_seq_q, Tensor cum_seq_k, int max_q, int max_k, float dropout_p, bool is_causal, Tensor philox_seed, Tensor philox_offset, *, float? scale=None) -> (Tensor, Tensor, Tensor)",
}


def _norm(s):
    return re.sub(r"=0\.0\b", "=0.", s).replace(" ", "")


def test_glue_defines_reference_schemas():
    torch_glue.load()
    for name, sig in REFERENCE_SCHEMAS.items():
        schema = str(getattr(torch.ops.b200_sdpa, name).default._schema)
        assert _norm(schema) == _norm(f"b200_sdpa::{name}{sig}"), schema
    assert torch.ops.b200_sdpa._launch_count() >= 0


def test_sdp_kernel_toggles_restore_state():
    before = (backends.flash_sdp_enabled(), backends.mem_efficient_sdp_enabled(), backends.math_sdp_enabled())
    with backends.sdp_kernel(enable_flash=True, enable_math=False, enable_mem_efficient=False):
        assert backends.flash_sdp_enabled() and not backends.math_sdp_enabled()
        assert not backends.mem_efficient_sdp_enabled()
    assert (backends.flash_sdp_enabled(), backends.mem_efficient_sdp_enabled(), backends.math_sdp_enabled()) == before
    assert int(backends.SDPBackend.FLASH_ATTENTION) == 1 and int(backends.SDPBackend.ERROR) == -1
