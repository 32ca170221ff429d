"""Builds and loads the dispatcher glue (csrc/torch_glue.cpp -> lib/libsdpa_b200_torch.so).

After ``load()``:
* ``torch.ops.b200_sdpa._scaled_dot_product_flash_attention`` (+ ``_backward``) and
  ``torch.ops.b200_sdpa._flash_attention_forward`` (+ ``_backward``) exist with the reference's
  schemas (codegen/mlu_functions.yaml:1313-1316) and differentiate through autograd.
* ``install_aten_overrides()`` additionally points the CUDA kernels of the same four ``aten``
  operators at this library, so ``F.scaled_dot_product_attention`` under the flash backend runs
  here. It is opt-in because it changes those operators for the whole process.
"""
from __future__ import annotations

import os
import subprocess
import sys

import torch

from . import _cabi, build as native_build

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "csrc", "torch_glue.cpp")
LIB = os.path.join(_cabi.LIB_DIR, "libsdpa_b200_torch.so")
_loaded = False


def build(verbose: bool = False) -> str:
    """g++ the glue against the installed torch and the C-ABI library (no GPU needed)."""
    # A process that already holds the C-ABI library must not re-link it underneath itself: the glue would
    # then load the new file as a second copy with its own state (error text, launch counter).
    if _cabi._lib is None:
        native_build.build_native()
    newest = max(os.path.getmtime(SRC), os.path.getmtime(os.path.join(os.path.dirname(HERE), "include", "sdpa_b200.h")))
    if os.path.exists(LIB) and os.path.getmtime(LIB) >= newest:
        return LIB
    from torch.utils import cpp_extension
    inc = [f"-I{p}" for p in cpp_extension.include_paths()]
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    inc.append(f"-I{cuda_home}/include")
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_API_INCLUDE_EXTENSION_H",
           *inc, SRC, "-o", LIB, f"-L{_cabi.LIB_DIR}", "-lsdpa_b200", f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-lc10",
           "-ltorch_cuda", "-lc10_cuda", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError("building the torch glue failed")
    return LIB


def _register_autograd() -> None:
    """Autograd formulas for the b200_sdpa operators: the forward saves q, k, v, out and the
    logsumexp, the backward is the matching *_backward operator (what upstream derivatives.yaml
    wires for the aten operators the reference registers)."""
    ns = torch.ops.b200_sdpa

    def dense_setup(ctx, inputs, keyword_only_inputs, output):
        query, key, value, dropout_p, is_causal, _dbg = inputs[:6]
        out, lse, cum_q, cum_k, max_q, max_k, seed, offset, _ = output
        ctx.save_for_backward(query, key, value, out, lse, cum_q, cum_k, seed, offset)
        ctx.args = (max_q, max_k, dropout_p, is_causal)
        ctx.scale = keyword_only_inputs.get("scale")

    def dense_backward(ctx, grad_out, *ignored):
        query, key, value, out, lse, cum_q, cum_k, seed, offset = ctx.saved_tensors
        max_q, max_k, dropout_p, is_causal = ctx.args
        dq, dk, dv = ns._scaled_dot_product_flash_attention_backward(grad_out, query, key, value, out, lse, cum_q, cum_k,
                                                                      max_q, max_k, dropout_p, is_causal, seed, offset,
                                                                      scale=ctx.scale)
        return dq, dk, dv, None, None, None

    def varlen_setup(ctx, inputs, keyword_only_inputs, output):
        query, key, value, cum_q, cum_k, max_q, max_k, dropout_p, is_causal, _dbg = inputs[:10]
        out, lse, seed, offset, _ = output
        ctx.save_for_backward(query, key, value, out, lse, cum_q, cum_k, seed, offset)
        ctx.args = (max_q, max_k, dropout_p, is_causal)
        ctx.scale = keyword_only_inputs.get("scale")

    def varlen_backward(ctx, grad_out, *ignored):
        query, key, value, out, lse, cum_q, cum_k, seed, offset = ctx.saved_tensors
        max_q, max_k, dropout_p, is_causal = ctx.args
        dq, dk, dv = ns._flash_attention_backward(grad_out, query, key, value, out, lse, cum_q, cum_k, max_q, max_k,
                                                  dropout_p, is_causal, seed, offset, scale=ctx.scale)
        return dq, dk, dv, None, None, None, None, None, None, None

    torch.library.register_autograd("b200_sdpa::_scaled_dot_product_flash_attention", dense_backward,
                                    setup_context=dense_setup)
    torch.library.register_autograd("b200_sdpa::_flash_attention_forward", varlen_backward, setup_context=varlen_setup)


def load() -> None:
    """Load the glue library (building it first if needed). Raises if it cannot be built."""
    global _loaded
    if _loaded:
        return
    build()
    _cabi.load()
    torch.ops.load_library(LIB)
    _register_autograd()
    _loaded = True


def install_aten_overrides() -> None:
    load()
    torch.ops.b200_sdpa._install_aten_overrides()


def remove_aten_overrides() -> None:
    if _loaded:
        torch.ops.b200_sdpa._remove_aten_overrides()


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv))
