"""Compile the CUDA library in-tree for sm_100a (nvcc cross-compiles without a GPU)."""
from __future__ import annotations

import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libtyr_b200_attn.so")
SOURCES = ["api.cu", "prefill_sm100.cu", "backward_sm100.cu", "decode_splitkv.cu", "check_fp32.cu", "qk_prologue.cu",
           "stalled_wait.cu"]
HEADERS = ["ptx_sm100.cuh", "mma_sync.cuh", "attn_internal.h", os.path.join("..", "..", "include", "tyr_b200_attn.h")]

# The reference's own nvcc flags for GPU=B200 (cc/Makefile:66-76) minus fast-math
# (the kernels ask for approximate ex2/lg2 explicitly where they want them) and
# minus the ThunderKittens define.
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-std=c++17", "-O3", "--expt-relaxed-constexpr", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared",
]


def nvcc_path() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the attention library cannot be built")
    return nvcc


def stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Build lib/libtyr_b200_attn.so if missing or older than its sources."""
    if not force and not stale():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [nvcc_path()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else [])
    cmd += ["-o", LIB_PATH] + [os.path.join(CSRC, f) for f in SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        print(res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force=True, verbose=True))
