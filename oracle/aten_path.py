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


def lse(q, k, v, is_causal: bool):
    """Natural-log LSE of the scaled scores, [B,Hq,Sq] fp32, from ATen's CPU flash kernel."""
    n_head, n_kv_head = q.shape[1], k.shape[1]
    if n_head != n_kv_head:
        rep = n_head // n_kv_head
        k = k.repeat_interleave(rep, 1)
        v = v.repeat_interleave(rep, 1)
    out = torch.ops.aten._scaled_dot_product_flash_attention_for_cpu(q, k, v, 0.0, is_causal)
    return out[1]
