import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# bf16 I/O against the fp32 CPU result (the north-star bars)
O_MAX_ABS = 2e-2
LSE_REL = 1e-3
CHECK_REL = 1e-5
# backward, bf16 I/O with P and dS rounded to bf16 before the matrix products (as the reference's
# own backward kernels do): max-abs error of each gradient relative to its largest entry
GRAD_REL_TO_MAX = 2e-2


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden():
    path = os.path.join(ROOT, "tests", "golden", "aten_sdpa.npz")
    data = np.load(path)
    names = sorted({k.split(".")[0] for k in data.files if "." in k})
    out = {}
    for n in names:
        case = {f: data[f"{n}.{f}"] for f in ("o", "lse", "meta")}
        if case["meta"].size < 8:      # [B, Hq, Hkv, Sq, Skv, D, causal, window]
            case["meta"] = np.append(case["meta"], 0)
        for f in ("q", "k", "v"):  # stored as bf16 bit patterns
            case[f] = (data[f"{n}.{f}"].astype(np.uint32) << 16).view(np.float32)
        out[n] = case
    return out


@pytest.fixture(scope="session")
def golden_backward():
    data = np.load(os.path.join(ROOT, "tests", "golden", "aten_backward.npz"))
    names = sorted({k.split(".")[0] for k in data.files if "." in k})
    out = {}
    for n in names:
        case = {f: data[f"{n}.{f}"] for f in ("d_q", "d_k", "d_v", "meta")}
        for f in ("q", "k", "v", "d_o"):  # stored as bf16 bit patterns
            case[f] = (data[f"{n}.{f}"].astype(np.uint32) << 16).view(np.float32)
        out[n] = case
    return out


@pytest.fixture(scope="session")
def built_lib():
    """The CUDA library, compiled if needed (nvcc cross-compiles without a GPU)."""
    from tyr_b200 import _lib, build
    build.build()
    return _lib.load()
