"""The reference's attention path on the CPU: the ATen operator its FFI calls.

Test infrastructure only.  Each function restates one `lean_torch_sdpa_*` entry
point of cc/src/tyr.cpp around `torch.nn.functional.scaled_dot_product_attention`
(the Python name of `torch::scaled_dot_product_attention`), including the
repeat_interleave GQA expansion that the reference performs inside the call.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def sdpa_4d(q, k, v, dropout_p: float = 0.0, is_causal: bool = True):
    """cc/src/tyr.cpp:2563-2589 (lean_torch_sdpa_4d)."""
    return F.scaled_dot_product_attention(q, k, v, None, dropout_p, is_causal)


def sdpa_gqa(q, k, v, dropout_p: float = 0.0, is_causal: bool = True, enable_gqa: bool = True):
    """cc/src/tyr.cpp:3913-3949 (lean_torch_sdpa_gqa); same body as ..._qkv at 4100-4133."""
    n_head, n_kv_head = q.shape[1], k.shape[1]
    if enable_gqa and n_head != n_kv_head and n_kv_head > 0:
        rep = n_head // n_kv_head
        k = k.repeat_interleave(rep, 1)
        v = v.repeat_interleave(rep, 1)
    return F.scaled_dot_product_attention(q, k, v, None, dropout_p, is_causal)


sdpa_gqa_qkv = sdpa_gqa


def sdpa_gqa_window(q, k, v, dropout_p: float = 0.0, is_causal: bool = True, enable_gqa: bool = True,
                    window_size: int = 1):
    """cc/src/tyr.cpp:3953-4018 (lean_torch_sdpa_gqa_window): explicit -inf/0 mask that hides
    future keys and keys `window_size` or more positions back, then SDPA with is_causal=false."""
    n_head, n_kv_head = q.shape[1], k.shape[1]
    if enable_gqa and n_head != n_kv_head and n_kv_head > 0:
        rep = n_head // n_kv_head
        k = k.repeat_interleave(rep, 1)
        v = v.repeat_interleave(rep, 1)
    seq = q.shape[2]
    row = torch.arange(seq).unsqueeze(1)
    col = torch.arange(seq).unsqueeze(0)
    combined = (col > row) | ((row - col) >= int(window_size))
    mask = torch.where(combined, torch.full((seq, seq), float("-inf"), dtype=q.dtype),
                       torch.zeros((seq, seq), dtype=q.dtype)).unsqueeze(0).unsqueeze(0)
    return F.scaled_dot_product_attention(q, k, v, mask, dropout_p, False)


def sdpa_gqa_mask(q, k, v, padding_mask, dropout_p: float = 0.0, is_causal: bool = True,
                  enable_gqa: bool = True):
    """cc/src/tyr.cpp:4024-4095 (lean_torch_sdpa_gqa_mask): padding_mask [batch, seq], 1 = valid
    key, 0 = padding; turned into a -inf/0 mask (with the causal mask when asked) for SDPA."""
    n_head, n_kv_head = q.shape[1], k.shape[1]
    if enable_gqa and n_head != n_kv_head and n_kv_head > 0:
        rep = n_head // n_kv_head
        k = k.repeat_interleave(rep, 1)
        v = v.repeat_interleave(rep, 1)
    seq = q.shape[2]
    key_mask = padding_mask.unsqueeze(1).unsqueeze(2)
    ninf = float("-inf")
    if is_causal:
        row = torch.arange(seq).unsqueeze(1)
        col = torch.arange(seq).unsqueeze(0)
        combined = (col > row).unsqueeze(0).unsqueeze(0) | (key_mask == 0)
        mask = torch.where(combined, torch.full((1, 1, seq, seq), ninf, dtype=q.dtype),
                           torch.zeros((1, 1, seq, seq), dtype=q.dtype))
    else:
        mask = torch.where(key_mask == 0, torch.full((1, 1, 1, seq), ninf, dtype=q.dtype),
                           torch.zeros((1, 1, 1, seq), dtype=q.dtype))
    return F.scaled_dot_product_attention(q, k, v, mask, dropout_p, False)


def sdpa_gqa_backward(q, k, v, d_o, is_causal: bool = True, window: int = 0, padding_mask=None):
    """Gradients LibTorch autograd gives the reference for its typed attention call:
    `output.backward(grad_output)` (cc/src/tyr.cpp:2111-2122) through lean_torch_sdpa_gqa
    (cc/src/tyr.cpp:3913-3949, repeat_interleave included), or through the windowed / padding-masked
    entry points when `window` / `padding_mask` is given.  Returns (d_q, d_k, d_v)."""
    q, k, v = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    if window:
        out = sdpa_gqa_window(q, k, v, 0.0, is_causal, True, window)
    elif padding_mask is not None:
        out = sdpa_gqa_mask(q, k, v, padding_mask, 0.0, is_causal, True)
    else:
        out = sdpa_gqa(q, k, v, 0.0, is_causal, True)
    out.backward(d_o)
    return q.grad, k.grad, v.grad


def lse(q, k, v, is_causal: bool):
    """Natural-log LSE of the scaled scores, [B,Hq,Sq] fp32, from ATen's CPU flash kernel."""
    n_head, n_kv_head = q.shape[1], k.shape[1]
    if n_head != n_kv_head:
        rep = n_head // n_kv_head
        k = k.repeat_interleave(rep, 1)
        v = v.repeat_interleave(rep, 1)
    out = torch.ops.aten._scaled_dot_product_flash_attention_for_cpu(q, k, v, 0.0, is_causal)
    return out[1]


def head_norm_rope_transpose(x, weight=None, cos=None, sin=None, eps: float = 1e-6):
    """The op chain Tyr runs on a projected [B,S,H,D] tensor before attention:
    applyHeadNorm (Tyr/Model/Qwen/Attention.lean:73-98), rotary.applyRotaryEmb
    (cc/src/tyr.cpp:3824-3861) and transpose_for_attention (cc/src/tyr.cpp:2402-2414)."""
    if weight is not None:
        var = (x * x).mean(-1, keepdim=True)
        x = x * torch.rsqrt(var + eps) * weight.reshape(1, 1, 1, -1)
    if cos is not None:
        d = x.shape[3] // 2
        x1, x2 = x[..., :d], x[..., d:]
        cb, sb = cos.unsqueeze(0).unsqueeze(2), sin.unsqueeze(0).unsqueeze(2)
        x = torch.cat([x1 * cb - x2 * sb, x1 * sb + x2 * cb], 3)
    return x.permute(0, 2, 1, 3).contiguous()


def slice_scatter_seq(cache, start: int, src):
    """data.sliceScatter along the sequence axis (cc/src/tyr.cpp:2261-2277): a new cache."""
    out = cache.clone()
    out[:, :, start:start + src.shape[2]].copy_(src)
    return out


def flux_rope_transpose(x, pe, weight=None, eps: float = 1e-6):
    """QKNorm.forward (Tyr/Model/Flux/QKNorm.lean:32-39) then flux.applyRope
    (Tyr/Model/Flux/RoPE.lean:71-96) on a projected [B,S,H,D] tensor, returned in the attention
    layout [B,H,S,D] (the transpose_for_attention of DoubleStreamBlock.lean:179-181).
    pe: [B, 1, S, D/2, 2, 2].  The op sequence of applyRopeAttn is kept: reshape to pairs, slice the
    two pair elements, expand, out = pe[..., 0] * x0 + pe[..., 1] * x1."""
    B, S, H, D = x.shape
    if weight is not None:
        var = (x * x).mean(-1, keepdim=True)
        x = x * torch.rsqrt(var + eps) * weight.reshape(1, 1, 1, -1)
    xa = x.permute(0, 2, 1, 3).contiguous().float()                    # transpose_for_attention, toFloat
    xr = xa.reshape(B, H, S, D // 2, 1, 2)
    x0 = xr[..., 0:1].reshape(B, H, S, D // 2, 1).expand(B, H, S, D // 2, 2)
    x1 = xr[..., 1:2].reshape(B, H, S, D // 2, 1).expand(B, H, S, D // 2, 2)
    pe0 = pe[..., 0:1].reshape(B, 1, S, D // 2, 2).expand(B, H, S, D // 2, 2)
    pe1 = pe[..., 1:2].reshape(B, 1, S, D // 2, 2).expand(B, H, S, D // 2, 2)
    return (pe0 * x0 + pe1 * x1).reshape(B, H, S, D)
