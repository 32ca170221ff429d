"""Builds the native code in-tree: torch_mlu_b200/lib/libsdpa_b200.so (C ABI + sm_100a kernels).

Run as ``python -m torch_mlu_b200.build``. nvcc cross-compiles for sm_100a, so no GPU is needed
to build. Objects are rebuilt only when a source or header is newer.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
OBJ_DIR = os.path.join(HERE, "build")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

SOURCES = ["sdpa_api.cu", "fwd_prefill_sm100.cu", "decode_splitkv.cu", "bwd_sm100.cu", "bwd_fused_sm100.cu", "merge_partials.cu",
           "dropout_mask.cu", "bias_transpose.cu", "d256_sm100.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-diag-suppress", "550",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC or put it on PATH)")


def _newest_header() -> float:
    paths = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    paths.append(os.path.join(INCLUDE, "sdpa_b200.h"))
    return max(os.path.getmtime(p) for p in paths)


def build_native(verbose: bool = False, force: bool = False) -> str:
    os.makedirs(LIB_DIR, exist_ok=True)
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()
    hdr = _newest_header()
    jobs = []
    objs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        objs.append(o)
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr):
            # SDPA_B200_NVCC_EXTRA: extra compile flags, e.g. -DSDPA_BWD_STAMPS for a profiling build
            cmd = [nvcc, *NVCC_FLAGS, *os.environ.get("SDPA_B200_NVCC_EXTRA", "").split(), "-I", INCLUDE, "-c", s, "-o", o]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {cmd[-3]}")

    with ThreadPoolExecutor(max_workers=4) as ex:
        list(ex.map(run, jobs))
    lib = os.path.join(LIB_DIR, "libsdpa_b200.so")
    if jobs or not os.path.exists(lib):
        run([nvcc, "-shared", "-o", lib, *objs])
    return lib


if __name__ == "__main__":
    print(build_native(verbose="-v" in sys.argv, force="-f" in sys.argv))
