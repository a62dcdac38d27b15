"""Build libspsattn.so in-tree with nvcc for sm_100a.

    python -m sps_b200.build [--force] [--verbose]

The shared library is the product: ``sps_b200`` loads it with ctypes and refuses
to work without it.  nvcc cross-compiles, so this runs on a machine without a GPU.
"""

from __future__ import annotations

import os
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libspsattn.so")
SOURCES = ["spsattn_api.cu"]
HEADERS = ["common.cuh", "mask.cuh", "prefill_sm100.cuh", "prefill_wide_sm100.cuh", "prefill_bwd_sm100.cuh", "prefill_aux.cuh", "decode.cuh", "decode_sm100.cuh",
           "kv_update.cuh", "model_glue.cuh", "rope.cuh", "cache_fill.cuh", os.path.join("..", "..", "include", "spsattn.h")]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > built for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not is_stale():
        return LIB_PATH
    cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "-shared", "-Xcompiler", "-fPIC", "--use_fast_math", "-o", LIB_PATH]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(CSRC, s) for s in SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stdout + res.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
