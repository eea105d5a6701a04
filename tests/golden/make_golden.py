"""Generate tests/golden/aten_sdpa.npz: outputs of the ATen operator the reference calls.

Run from the repo root:  python tests/golden/make_golden.py
Every case calls `oracle.aten_path` (a restatement of the `lean_torch_sdpa_*`
forwards of cc/src/tyr.cpp around torch's scaled_dot_product_attention) on fp32
tensors whose values are bf16-representable, the reference's own fixture
convention (Examples/GPU/RunFlashAttn.lean:30-36).  torch version is recorded.
"""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "..", ".."))
from oracle import aten_path  # noqa: E402

# name: (entry point, B, Hq, Hkv, Sq, Skv, D, causal, rmsnorm_qk)
CASES = {
    "gpt_mha_causal": ("sdpa_4d", 2, 2, 2, 40, 40, 64, True, False),
    "qwen_gqa_causal": ("sdpa_gqa", 1, 2, 1, 65, 65, 128, True, True),
    "flux_mha_full": ("sdpa_4d", 1, 1, 1, 96, 96, 128, False, True),
    "decode_gqa_step": ("sdpa_gqa_qkv", 2, 4, 1, 1, 77, 128, False, False),
    "qkv_causal_topleft": ("sdpa_gqa_qkv", 1, 2, 1, 5, 9, 64, True, False),
    "tile_edge_129": ("sdpa_gqa", 1, 2, 1, 129, 129, 64, True, False),
}


def rms(x):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6)


def main():
    out = {"torch_version": np.array(torch.__version__)}
    for i, (name, (fn, B, Hq, Hkv, Sq, Skv, D, causal, norm)) in enumerate(CASES.items()):
        g = torch.Generator(device="cpu").manual_seed(1000 + i)
        q = torch.randn(B, Hq, Sq, D, generator=g)
        k = torch.randn(B, Hkv, Skv, D, generator=g)
        v = torch.randn(B, Hkv, Skv, D, generator=g)
        if norm:
            q, k = rms(q), rms(k)
        q, k, v = (t.bfloat16().float() for t in (q, k, v))
        if fn == "sdpa_4d":
            o = aten_path.sdpa_4d(q, k, v, 0.0, causal)
        else:
            o = getattr(aten_path, fn)(q, k, v, 0.0, causal, True)
        lse = aten_path.lse(q, k, v, causal)
        # inputs are bf16-representable: store the upper 16 bits only
        for key, t in (("q", q), ("k", k), ("v", v)):
            out[f"{name}.{key}"] = (t.numpy().view(np.uint32) >> 16).astype(np.uint16)
        for key, t in (("o", o), ("lse", lse)):
            out[f"{name}.{key}"] = t.numpy()
        out[f"{name}.meta"] = np.array([B, Hq, Hkv, Sq, Skv, D, int(causal)])
    path = os.path.join(os.path.dirname(__file__), "aten_sdpa.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
