"""Generate tests/golden/aten_sdpa.npz: outputs of the ATen operator the reference calls.

Run from the repo root:  python tests/golden/make_golden.py [sdpa] [prologue] [keymask] [backward] [fluxrope]
(no argument: all of them).
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
    # sliding window (lean_torch_sdpa_gqa_window); the window size rides in WINDOWS below
    "window_7": ("sdpa_gqa_window", 1, 2, 1, 50, 50, 64, True, False),
    "window_140": ("sdpa_gqa_window", 1, 1, 1, 260, 260, 64, True, True),
}
WINDOWS = {"window_7": 7, "window_140": 140}


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
        win = WINDOWS.get(name, 0)
        if fn == "sdpa_4d":
            o = aten_path.sdpa_4d(q, k, v, 0.0, causal)
        elif win:
            o = aten_path.sdpa_gqa_window(q, k, v, 0.0, causal, True, win)
        else:
            o = getattr(aten_path, fn)(q, k, v, 0.0, causal, True)
        # ATen returns no LSE for a masked call: windowed cases store zeros and pin O only
        lse = aten_path.lse(q, k, v, causal) if not win else torch.zeros(B, Hq, Sq)
        # inputs are bf16-representable: store the upper 16 bits only
        for key, t in (("q", q), ("k", k), ("v", v)):
            out[f"{name}.{key}"] = (t.numpy().view(np.uint32) >> 16).astype(np.uint16)
        for key, t in (("o", o), ("lse", lse)):
            out[f"{name}.{key}"] = t.numpy()
        out[f"{name}.meta"] = np.array([B, Hq, Hkv, Sq, Skv, D, int(causal), win])
    path = os.path.join(os.path.dirname(__file__), "aten_sdpa.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


def main_keymask():
    """tests/golden/aten_keymask.npz: lean_torch_sdpa_gqa_mask restated with torch (padding mask)."""
    g = torch.Generator(device="cpu").manual_seed(3000)
    B, Hq, Hkv, S, D = 2, 1, 1, 130, 64
    q, k, v = (torch.randn(B, h, S, D, generator=g).bfloat16().float() for h in (Hq, Hkv, Hkv))
    m = torch.ones(B, S)
    m[0, 90:] = 0           # right padding
    m[1, 20:45] = 0         # a hole
    out = {"mask": m.numpy().astype(np.uint8), "torch_version": np.array(torch.__version__)}
    for key, t in (("q", q), ("k", k), ("v", v)):
        out[key] = (t.numpy().view(np.uint32) >> 16).astype(np.uint16)
    out["o_causal"] = aten_path.sdpa_gqa_mask(q, k, v, m, 0.0, True, True).numpy()
    out["o_full"] = aten_path.sdpa_gqa_mask(q, k, v, m, 0.0, False, True).numpy()
    path = os.path.join(os.path.dirname(__file__), "aten_keymask.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


def main_prologue():
    """tests/golden/aten_prologue.npz: the reference's op chain before attention (per-head
    RMSNorm, rotary embedding, transpose, cache slice_scatter) run with torch on fp32."""
    g = torch.Generator(device="cpu").manual_seed(2000)
    B, S, H, D, cap, start = 2, 3, 2, 128, 16, 5
    x = torch.randn(B, S, H, D, generator=g).bfloat16().float()
    w = (torch.rand(D, generator=g) + 0.5)
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, D // 2).float() / (D // 2)))
    ang = torch.arange(cap).float()[:, None] * inv_freq[None]
    cos, sin = ang.cos(), ang.sin()
    y = aten_path.head_norm_rope_transpose(x, w, cos[start:start + S], sin[start:start + S], 1e-6)
    cache = torch.randn(B, H, cap, D, generator=g).bfloat16().float()
    new_cache = aten_path.slice_scatter_seq(cache, start, y)
    out = {"x": x.numpy(), "w": w.numpy(), "cos": cos.numpy(), "sin": sin.numpy(),
           "cache": cache.numpy(), "new_cache": new_cache.numpy(), "start": np.array(start),
           "torch_version": np.array(torch.__version__)}
    path = os.path.join(os.path.dirname(__file__), "aten_prologue.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


def main_fluxrope():
    """tests/golden/aten_flux_rope.npz: QK-norm + Flux's interleaved rotary + transpose with torch
    on fp32 (the chain before the joint attention of DoubleStreamBlock.lean:163-181)."""
    g = torch.Generator(device="cpu").manual_seed(2100)
    B, S, H, D = 2, 5, 3, 128
    x = torch.randn(B, S, H, D, generator=g).bfloat16().float()
    w = (torch.rand(D, generator=g) + 0.5)
    # a rotation table per batch element and position: [[cos, -sin], [sin, cos]] per pair
    ang = torch.rand(B, 1, S, D // 2, generator=g) * 6.0
    pe = torch.stack([torch.stack([ang.cos(), -ang.sin()], -1), torch.stack([ang.sin(), ang.cos()], -1)], -2)
    y = aten_path.flux_rope_transpose(x, pe, w, 1e-6)
    out = {"x": x.numpy(), "w": w.numpy(), "pe": pe.numpy(), "y": y.numpy(),
           "torch_version": np.array(torch.__version__)}
    path = os.path.join(os.path.dirname(__file__), "aten_flux_rope.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


# name: (B, Hq, Hkv, Sq, Skv, D, causal)
BACKWARD_CASES = {
    "mha_causal": (1, 2, 2, 40, 40, 64, True),
    "gqa_causal": (1, 2, 1, 130, 130, 64, True),
    "gqa_full_ragged": (1, 2, 1, 30, 140, 128, False),
    "qkv_causal_topleft": (1, 2, 1, 135, 50, 64, True),
}


def main_backward():
    """tests/golden/aten_backward.npz: gradients from torch autograd through the restated
    lean_torch_sdpa_gqa (the derivative the reference's autograd.backward supplies)."""
    out = {"torch_version": np.array(torch.__version__)}
    for i, (name, (B, Hq, Hkv, Sq, Skv, D, causal)) in enumerate(BACKWARD_CASES.items()):
        g = torch.Generator(device="cpu").manual_seed(4000 + i)
        q = torch.randn(B, Hq, Sq, D, generator=g).bfloat16().float()
        k = torch.randn(B, Hkv, Skv, D, generator=g).bfloat16().float()
        v = torch.randn(B, Hkv, Skv, D, generator=g).bfloat16().float()
        d_o = torch.randn(B, Hq, Sq, D, generator=g).bfloat16().float()
        d_q, d_k, d_v = aten_path.sdpa_gqa_backward(q, k, v, d_o, causal)
        for key, t in (("q", q), ("k", k), ("v", v), ("d_o", d_o)):
            out[f"{name}.{key}"] = (t.numpy().view(np.uint32) >> 16).astype(np.uint16)
        for key, t in (("d_q", d_q), ("d_k", d_k), ("d_v", d_v)):
            out[f"{name}.{key}"] = t.numpy()
        out[f"{name}.meta"] = np.array([B, Hq, Hkv, Sq, Skv, D, int(causal)])
    path = os.path.join(os.path.dirname(__file__), "aten_backward.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    jobs = {"sdpa": main, "prologue": main_prologue, "keymask": main_keymask, "backward": main_backward,
            "fluxrope": main_fluxrope}
    for name in (sys.argv[1:] or list(jobs)):
        jobs[name]()
