"""ctypes loader for oracle/libsdpa_ref.so (plain-C fp64 restatement). TEST INFRASTRUCTURE ONLY."""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libsdpa_ref.so")


def build() -> str:
    subprocess.run(["make", "-C", HERE, "-s"], check=True)
    return LIB


def _lib():
    if not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(os.path.join(HERE, "sdpa_ref.c")):
        build()
    return ctypes.CDLL(LIB)


def _f32(t):
    return np.ascontiguousarray(t.detach().float().cpu().numpy(), dtype=np.float32)


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def forward(q, k, v, *, causal=False, scale=None):
    lib = _lib()
    qa, ka, va = _f32(q), _f32(k), _f32(v)
    B, Hq, Lq, D = qa.shape
    Hkv, Lk = ka.shape[1], ka.shape[2]
    sc = float(scale) if scale is not None else 1.0 / np.sqrt(D)
    out = np.empty_like(qa)
    lse = np.empty((B, Hq, Lq), dtype=np.float32)
    lib.sdpa_ref_forward(_p(qa), _p(ka), _p(va), _p(out), _p(lse), B, Hq, Hkv, Lq, Lk, D, ctypes.c_float(sc), int(causal))
    return torch.from_numpy(out), torch.from_numpy(lse)


def backward(q, k, v, dout, *, causal=False, scale=None):
    lib = _lib()
    qa, ka, va, da = _f32(q), _f32(k), _f32(v), _f32(dout)
    B, Hq, Lq, D = qa.shape
    Hkv, Lk = ka.shape[1], ka.shape[2]
    assert D <= 512
    sc = float(scale) if scale is not None else 1.0 / np.sqrt(D)
    dq, dk, dv = np.empty_like(qa), np.empty_like(ka), np.empty_like(va)
    lib.sdpa_ref_backward(_p(qa), _p(ka), _p(va), _p(da), _p(dq), _p(dk), _p(dv), B, Hq, Hkv, Lq, Lk, D,
                          ctypes.c_float(sc), int(causal))
    return torch.from_numpy(dq), torch.from_numpy(dk), torch.from_numpy(dv)
