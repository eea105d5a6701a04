"""Tyr's typed attention calls, served by the sm_100a kernels.

Names and defaults follow the Lean declarations:
  scaled_dot_product_attention        Tyr/Torch.lean:663-671   (is_causal := true)
  scaledDotProductAttentionGQA        Tyr/Torch.lean:1058-1067 (enable_gqa := false)
  scaledDotProductAttentionGQAQKV     Tyr/Torch.lean:1069-1082
Each is a pure function returning a new tensor, like the `T #[b,h,s,d]` result of
the Lean call.  `attentionFwd` is the launcher-style form (caller may pass the
outputs, LSE returned) and `flashDecode` the ragged single-token decode.

Tensors are torch CUDA tensors; only their data pointers, sizes and strides cross
the C ABI, and the launch goes on torch's current stream, which is what
`torch.cuda_current_stream` returns to Tyr (cc/src/tyr.cpp:4314-4331).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence, Tuple

import torch

from . import _lib
from ._lib import AttnError, BackwardArgs, DecodeArgs, PrefillArgs, PrologueArgs, check


def _stream_ptr(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _require_cuda(*ts: torch.Tensor) -> None:
    # the launcher checks of Tyr/GPU/Codegen/Attribute.lean:333-336, as exceptions
    for t in ts:
        if not t.is_cuda:
            raise ValueError("tensor must be on a CUDA device")
        if t.dim() > 4:
            raise ValueError("tensor rank must be <= 4")
        if t.stride(-1) != 1:
            raise ValueError("tensor must have unit stride on the head dimension")


def _fill_prefill(q, k, v, o, lse, is_causal, scale, check_mode, window_size=0, key_mask=None) -> PrefillArgs:
    B, Hq, Sq, D = q.shape
    Bk, Hkv, Skv, Dk = k.shape
    if v.shape != k.shape or Bk != B or Dk != D or o.shape != q.shape:
        raise ValueError(f"shape mismatch: q {tuple(q.shape)} k {tuple(k.shape)} v {tuple(v.shape)}")
    if q.dtype != k.dtype or q.dtype != v.dtype or q.dtype != o.dtype:
        raise ValueError("q, k, v and out must share one dtype")
    if q.dtype == torch.bfloat16:
        dtype = _lib.TYR_ATTN_BF16
    elif q.dtype == torch.float32:
        dtype = _lib.TYR_ATTN_F32
    else:
        raise ValueError("dtype must be bfloat16 (float32 in check mode)")
    a = PrefillArgs()
    a.q, a.k, a.v, a.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    a.lse = lse.data_ptr() if lse is not None else None
    a.batch, a.n_head, a.n_kv_head, a.q_seq, a.kv_seq, a.head_dim = B, Hq, Hkv, Sq, Skv, D
    for name, t in (("q_stride", q), ("k_stride", k), ("v_stride", v), ("o_stride", o)):
        getattr(a, name)[:] = [t.stride(0), t.stride(1), t.stride(2)]
    a.dtype, a.is_causal, a.scale, a.check_mode = dtype, int(bool(is_causal)), float(scale or 0.0), int(bool(check_mode))
    a.window_size = int(window_size)
    if key_mask is not None:
        a.key_mask, a.key_mask_stride = key_mask.data_ptr(), key_mask.stride(0)
    else:
        a.key_mask, a.key_mask_stride = None, 0
    return a


def attentionFwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, is_causal: bool = True,
                 scale: Optional[float] = None, out: Optional[torch.Tensor] = None,
                 lse: Optional[torch.Tensor] = None, return_lse: bool = True,
                 check_mode: bool = False, window_size: int = 0,
                 key_mask: Optional[torch.Tensor] = None,
                 workspace=None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """O = softmax(Q K^T * scale + causal) V and the per-row LSE.

    q [B,Hq,Sq,D]; k, v [B,Hkv,Skv,D] (Hq % Hkv == 0, query head h reads KV head
    h // (Hq/Hkv) as repeat_interleave does, cc/src/tyr.cpp:3931-3938).  Strided
    views are accepted (unit inner stride), e.g. the KV-cache slice of
    Tyr/Model/Qwen/Attention.lean:195-196.  `check_mode` runs the fp32-FMA kernel.
    `window_size` > 0 adds the causal sliding window of lean_torch_sdpa_gqa_window
    (cc/src/tyr.cpp:3986-3996): key j is visible to query i only if j <= i and i - j < window_size.
    `key_mask` (uint8 / bool CUDA tensor [batch, kv_seq], 0 = padding key) hides padding keys
    from every query, the key side of lean_torch_sdpa_gqa_mask (cc/src/tyr.cpp:4063-4086).
    Launcher convention of Examples/GPU/RunFlashAttn.lean:68-81: outputs may be
    pre-allocated by the caller and are written in place.
    `workspace`: a caller-kept uint8 CUDA tensor of `prefill_workspace_bytes(...)` bytes for the
    key-split of a half-empty last round; when the call would split, one is allocated if none is given
    (`workspace=False`: never split).
    """
    _require_cuda(q, k, v)
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("q, k, v must be [batch, heads, seq, head_dim]")
    if out is None:
        out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    if lse is None and return_lse:
        lse = torch.empty(q.shape[:3], dtype=torch.float32, device=q.device)
    if lse is not None and (lse.dtype != torch.float32 or not lse.is_contiguous()
                            or tuple(lse.shape) != tuple(q.shape[:3])):
        raise ValueError("lse must be a contiguous float32 [batch, n_head, q_seq] tensor")
    if key_mask is not None:
        if key_mask.dtype == torch.bool:
            key_mask = key_mask.view(torch.uint8)
        if (not key_mask.is_cuda or key_mask.dtype != torch.uint8 or key_mask.dim() != 2
                or key_mask.stride(1) != 1 or tuple(key_mask.shape) != (k.shape[0], k.shape[2])):
            raise ValueError("key_mask must be a uint8/bool CUDA tensor [batch, kv_seq]")
    a = _fill_prefill(q, k, v, out, lse, is_causal, scale, check_mode, window_size, key_mask)
    L = _lib.load()
    with torch.cuda.device(q.device):
        # only unmasked, non-causal calls are ever split: no query for the others
        may_split = workspace is not False and not is_causal and window_size == 0 and key_mask is None and not check_mode
        need = int(L.tyr_b200_attn_prefill_workspace_bytes(ctypes.byref(a))) if may_split else 0
        if need > 0:
            if workspace is None:
                workspace = torch.empty(need, dtype=torch.uint8, device=q.device)
            if (workspace.dtype != torch.uint8 or not workspace.is_contiguous() or workspace.device != q.device
                    or workspace.data_ptr() % 256 != 0):
                raise ValueError("workspace must be a contiguous uint8 CUDA tensor on q's device, 256-byte aligned")
            a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel()
        check(L.tyr_b200_attn_prefill(ctypes.byref(a), _stream_ptr(q)))
    return out, lse


def prefill_workspace_bytes(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, is_causal: bool = True) -> int:
    """Bytes of `workspace` with which `attentionFwd` on these tensors would split its last round (0: it would not)."""
    a = _fill_prefill(q, k, v, q, None, is_causal, None, False)  # only shapes and strides are looked at
    with torch.cuda.device(q.device):
        return max(int(_lib.load().tyr_b200_attn_prefill_workspace_bytes(ctypes.byref(a))), 0)


def attentionBwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor, lse: torch.Tensor,
                 d_o: torch.Tensor, is_causal: bool = True, scale: Optional[float] = None,
                 workspace: Optional[torch.Tensor] = None, window_size: int = 0,
                 key_mask: Optional[torch.Tensor] = None
                 ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """dQ, dK, dV of `attentionFwd` from dO, the forward's inputs, its output and its LSE.

    The gradient LibTorch autograd produces for the typed attention call in the reference
    (`autograd.backward`, Tyr/Torch.lean:742 -> cc/src/tyr.cpp:2111-2122), computed with the
    formulation of Tyr/GPU/Kernels/MhaH100.lean:196-344.  dK and dV of a KV head are summed over
    the query heads that share it.  `workspace` may be a caller-kept float32 CUDA tensor of at
    least `backward_workspace_bytes(...) / 4` elements; one is allocated otherwise.
    `window_size` and `key_mask` are those of the forward call (sliding window / padding keys).
    """
    _require_cuda(q, k, v, o, d_o, lse)
    B, Hq, Sq, D = q.shape
    Bk, Hkv, Skv, Dk = k.shape
    if (v.shape != k.shape or Bk != B or Dk != D or o.shape != q.shape or d_o.shape != q.shape
            or tuple(lse.shape) != (B, Hq, Sq)):
        raise ValueError("shape mismatch among q, k, v, o, d_o, lse")
    if any(t.dtype != torch.bfloat16 for t in (q, k, v, o, d_o)):
        raise ValueError("q, k, v, o, d_o must be bfloat16")
    if lse.dtype != torch.float32 or not lse.is_contiguous():
        raise ValueError("lse must be a contiguous float32 [batch, n_head, q_seq] tensor")
    L = _lib.load()
    need = int(L.tyr_b200_attn_backward_workspace_bytes(B, Hq, Sq))
    if workspace is None:
        workspace = torch.empty(need // 4, dtype=torch.float32, device=q.device)
    if workspace.dtype != torch.float32 or not workspace.is_contiguous() or workspace.numel() * 4 < need:
        raise ValueError("workspace must be a contiguous float32 CUDA tensor of the required size")
    d_q, d_k, d_v = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    a = BackwardArgs()
    a.q, a.k, a.v, a.o, a.d_o, a.lse = (t.data_ptr() for t in (q, k, v, o, d_o, lse))
    a.d_q, a.d_k, a.d_v = d_q.data_ptr(), d_k.data_ptr(), d_v.data_ptr()
    a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel() * 4
    a.batch, a.n_head, a.n_kv_head, a.q_seq, a.kv_seq, a.head_dim = B, Hq, Hkv, Sq, Skv, D
    for name, t in (("q_stride", q), ("k_stride", k), ("v_stride", v), ("o_stride", o), ("do_stride", d_o),
                    ("dq_stride", d_q), ("dk_stride", d_k), ("dv_stride", d_v)):
        getattr(a, name)[:] = [t.stride(0), t.stride(1), t.stride(2)]
    a.dtype, a.is_causal, a.scale = _lib.TYR_ATTN_BF16, int(bool(is_causal)), float(scale or 0.0)
    a.window_size = int(window_size)
    if key_mask is not None:
        if key_mask.dtype == torch.bool:
            key_mask = key_mask.view(torch.uint8)
        if (not key_mask.is_cuda or key_mask.dtype != torch.uint8 or key_mask.dim() != 2
                or key_mask.stride(1) != 1 or tuple(key_mask.shape) != (B, Skv)):
            raise ValueError("key_mask must be a uint8/bool CUDA tensor [batch, kv_seq]")
        a.key_mask, a.key_mask_stride = key_mask.data_ptr(), key_mask.stride(0)
    else:
        a.key_mask, a.key_mask_stride = None, 0
    with torch.cuda.device(q.device):
        check(L.tyr_b200_attn_backward(ctypes.byref(a), _stream_ptr(q)))
    return d_q, d_k, d_v


def _sdpa(q, k, v, dropout_p, is_causal, enable_gqa):
    if dropout_p != 0.0:
        # the C ABI refuses dropout; a Tyr build keeps its LibTorch call for that case
        raise AttnError(-6)
    if not enable_gqa and q.shape[1] != k.shape[1]:
        raise AttnError(-2)
    out, _ = attentionFwd(q, k, v, is_causal=is_causal, return_lse=False)
    return out


def scaled_dot_product_attention(query, key, value, dropout_p: float = 0.0, is_causal: bool = True):
    """Tyr/Torch.lean:663-671 -> lean_torch_sdpa_4d (cc/src/tyr.cpp:2563-2589)."""
    return _sdpa(query, key, value, dropout_p, is_causal, False)


def scaledDotProductAttentionGQA(query, key, value, dropout_p: float = 0.0, is_causal: bool = True,
                                 enable_gqa: bool = False):
    """Tyr/Torch.lean:1058-1067 -> lean_torch_sdpa_gqa (cc/src/tyr.cpp:3913-3949)."""
    if query.shape[2] != key.shape[2]:
        raise ValueError("scaledDotProductAttentionGQA needs q_seq == kv_seq; use ...GQAQKV")
    return _sdpa(query, key, value, dropout_p, is_causal, enable_gqa)


def scaledDotProductAttentionGQAQKV(query, key, value, dropout_p: float = 0.0, is_causal: bool = True,
                                    enable_gqa: bool = False):
    """Tyr/Torch.lean:1069-1082 -> lean_torch_sdpa_gqa_qkv (cc/src/tyr.cpp:4100-4133)."""
    return _sdpa(query, key, value, dropout_p, is_causal, enable_gqa)


def scaledDotProductAttentionGQAWindow(query, key, value, dropout_p: float = 0.0, is_causal: bool = True,
                                       enable_gqa: bool = False, window_size: int = 1):
    """Tyr/Torch.lean:1084-1101 -> lean_torch_sdpa_gqa_window (cc/src/tyr.cpp:3953-4018).
    As in the reference, the mask is always causal | window whatever `is_causal` says."""
    if dropout_p != 0.0:
        raise AttnError(-6)
    if (not enable_gqa and query.shape[1] != key.shape[1]) or window_size <= 0:
        raise AttnError(-2)
    if query.shape[2] != key.shape[2]:
        raise ValueError("scaledDotProductAttentionGQAWindow needs q_seq == kv_seq")
    out, _ = attentionFwd(query, key, value, is_causal=True, return_lse=False, window_size=window_size)
    return out


def scaledDotProductAttentionGQAMask(query, key, value, attn_mask, dropout_p: float = 0.0,
                                     is_causal: bool = True, enable_gqa: bool = False):
    """Tyr/Torch.lean:1103-1118 -> lean_torch_sdpa_gqa_mask (cc/src/tyr.cpp:4024-4095).
    attn_mask [batch, seq]: non-zero = valid key, 0 = padding (any numeric or bool dtype)."""
    if dropout_p != 0.0:
        raise AttnError(-6)
    if not enable_gqa and query.shape[1] != key.shape[1]:
        raise AttnError(-2)
    if query.shape[2] != key.shape[2]:
        raise ValueError("scaledDotProductAttentionGQAMask needs q_seq == kv_seq")
    km = (attn_mask != 0).to(torch.uint8).contiguous()   # one byte per key for the C ABI
    out, _ = attentionFwd(query, key, value, is_causal=is_causal, return_lse=False, key_mask=km)
    return out


def sdpa_host(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, is_causal: bool = True,
              out: Optional[torch.Tensor] = None, lse: Optional[torch.Tensor] = None,
              device: int = 0) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Host-buffer call: q/k/v/out are CPU tensors (pinned for full copy speed)."""
    for t in (q, k, v):
        if t.is_cuda or not t.is_contiguous():
            raise ValueError("sdpa_host takes contiguous CPU tensors")
    if out is None:
        out = torch.empty(q.shape, dtype=q.dtype).pin_memory()
    a = _fill_prefill(q, k, v, out, lse, is_causal, None, False)
    check(_lib.load().tyr_b200_attn_prefill_host(ctypes.byref(a), device))
    return out, lse


class DecodePlan:
    """Device-side description of a ragged KV cache for `flashDecode`.

    Holds the pointer and length arrays and the split-KV workspace so that the
    per-token call allocates nothing.  `k_list[b]`, `v_list[b]` are
    [n_kv_head, len_b, head_dim] bf16 tensors (contiguous or with a head stride).
    """

    def __init__(self, k_list: Sequence[torch.Tensor], v_list: Sequence[torch.Tensor],
                 n_head: int, max_splits: int = 64):
        if len(k_list) == 0 or len(k_list) != len(v_list):
            raise ValueError("need one K and one V tensor per sequence")
        dev = k_list[0].device
        self.device, self.batch, self.n_head = dev, len(k_list), n_head
        self.n_kv_head, _, self.head_dim = k_list[0].shape
        lens, kp, vp, hs = [], [], [], []
        for kt, vt in zip(k_list, v_list):
            _require_cuda(kt, vt)
            if kt.shape != vt.shape or kt.dtype != torch.bfloat16 or kt.stride() != vt.stride():
                raise ValueError("K and V of a sequence must match in shape, stride and be bf16")
            if kt.stride(1) != self.head_dim:
                raise ValueError("keys of one head must be contiguous rows")
            # the kernel reads rows with 16-byte copies straight from these pointers
            if kt.data_ptr() % 16 or vt.data_ptr() % 16 or kt.stride(0) % 8:
                raise ValueError("each K/V block must be 16-byte aligned with a head stride that is a multiple of 8")
            if kt.shape[1] < 1:
                raise ValueError("every sequence needs at least one cached key")
            lens.append(kt.shape[1]); kp.append(kt.data_ptr()); vp.append(vt.data_ptr()); hs.append(kt.stride(0))
        self._keep = (list(k_list), list(v_list))
        self.max_kv_seq = max(lens)
        self.lens_host = lens
        self.total_kv_len = int(sum(lens))
        self.kv_lens = torch.tensor(lens, dtype=torch.int32, device=dev)
        self.k_ptrs = torch.tensor(kp, dtype=torch.int64, device=dev)
        self.v_ptrs = torch.tensor(vp, dtype=torch.int64, device=dev)
        self.head_strides = torch.tensor(hs, dtype=torch.int64, device=dev)
        self.max_splits = max_splits
        nbytes = _lib.load().tyr_b200_attn_decode_workspace_bytes(self.batch, n_head, self.head_dim,
                                                                  self.max_kv_seq, max_splits)
        self.workspace = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dev)
        self.workspace_bytes = nbytes


def _fill_decode(q3, plan: DecodePlan, out, lse, scale) -> DecodeArgs:
    """Arguments of a ragged decode call over `plan`, without the workspace."""
    a = DecodeArgs()
    a.q, a.o, a.lse = q3.data_ptr(), out.data_ptr(), (lse.data_ptr() if lse is not None else None)
    a.k = a.v = None
    a.k_ptrs, a.v_ptrs = plan.k_ptrs.data_ptr(), plan.v_ptrs.data_ptr()
    a.kv_lens, a.kv_head_strides = plan.kv_lens.data_ptr(), plan.head_strides.data_ptr()
    a.batch, a.n_head, a.n_kv_head = plan.batch, plan.n_head, plan.n_kv_head
    a.max_kv_seq, a.head_dim = plan.max_kv_seq, plan.head_dim
    a.q_stride[:] = [q3.stride(0), q3.stride(1)]
    a.o_stride[:] = [out.stride(0), out.stride(1)]
    a.k_stride[:] = [0, 0, plan.head_dim]
    a.v_stride[:] = [0, 0, plan.head_dim]
    a.scale, a.max_splits = float(scale or 0.0), plan.max_splits
    a.total_kv_len = plan.total_kv_len     # the host built the plan from these lengths: let the launch size its chunks by them
    return a


def flashDecode(q: torch.Tensor, plan: DecodePlan, scale: Optional[float] = None,
                out: Optional[torch.Tensor] = None, lse: Optional[torch.Tensor] = None,
                return_lse: bool = True):
    """One query token per sequence over the ragged cache of `plan`.

    q [B, n_head, head_dim] (or [B, n_head, 1, head_dim]) bf16.  Same result as
    scaledDotProductAttentionGQAQKV(q[b:b+1], K_b, V_b, 0.0, false, true) for each b,
    the call QwenAttention.forwardStep makes (Tyr/Model/Qwen/Attention.lean:198-200).
    """
    squeeze = q.dim() == 4
    q3 = q[:, :, 0, :] if squeeze else q
    _require_cuda(q3)
    if q3.dtype != torch.bfloat16 or q3.shape != (plan.batch, plan.n_head, plan.head_dim):
        raise ValueError("q must be bf16 [batch, n_head, head_dim]")
    if out is None:
        out = torch.empty((plan.batch, plan.n_head, plan.head_dim), dtype=q.dtype, device=q.device)
    if lse is None and return_lse:
        lse = torch.empty((plan.batch, plan.n_head), dtype=torch.float32, device=q.device)
    a = _fill_decode(q3, plan, out, lse, scale)
    a.workspace, a.workspace_bytes = plan.workspace.data_ptr(), plan.workspace_bytes
    with torch.cuda.device(q.device):
        check(_lib.load().tyr_b200_attn_decode(ctypes.byref(a), _stream_ptr(q)))
    if squeeze:
        return out.unsqueeze(2), (lse.unsqueeze(2) if lse is not None else None)
    return out, lse


def flashDecodeStatic(q: torch.Tensor, plan: DecodePlan, scale: Optional[float] = None,
                      out: Optional[torch.Tensor] = None, lse: Optional[torch.Tensor] = None):
    """`flashDecode` for callers that may not allocate device memory while decoding.

    Some hosts of this operator cannot call cudaMalloc in their token loop: their
    memory pool already owns the device, or an allocation's device-wide
    synchronisation would stall the loop.  This call goes through
    tyr_b200_attn_decode_static, which keeps the split-KV scratch in a fixed
    16 MiB array inside the library instead of `plan.workspace`, so the library
    allocates nothing; pass `out` and `lse` to keep this wrapper allocation-free too.
    Shapes whose scratch would not fit raise AttnError (size beyond the supported
    maximum).  All calls on one device share that array: keep them on one stream.
    The first call on a device looks the array up and should come before any
    stream capture.
    """
    q3 = q[:, :, 0, :] if q.dim() == 4 else q
    _require_cuda(q3)
    if q3.dtype != torch.bfloat16 or q3.shape != (plan.batch, plan.n_head, plan.head_dim):
        raise ValueError("q must be bf16 [batch, n_head, head_dim]")
    if out is None:
        out = torch.empty((plan.batch, plan.n_head, plan.head_dim), dtype=q.dtype, device=q.device)
    if lse is None:
        lse = torch.empty((plan.batch, plan.n_head), dtype=torch.float32, device=q.device)
    a = _fill_decode(q3, plan, out, lse, scale)
    a.workspace, a.workspace_bytes = None, 0      # ignored: the library's own array is used
    with torch.cuda.device(q.device):
        check(_lib.load().tyr_b200_attn_decode_static(ctypes.byref(a), _stream_ptr(q)))
    return out, lse


def flashDecodeDense(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     kv_lens: Optional[torch.Tensor] = None, kv_len: Optional[int] = None,
                     scale: Optional[float] = None, workspace: Optional[torch.Tensor] = None,
                     max_splits: int = 64):
    """Decode over Tyr's dense KVCache layout [batch, n_kv_head, cap, head_dim]
    (Tyr/Model/Qwen/Attention.lean:54-68).  `kv_len` plays the cache's shared `seq`
    counter; `kv_lens` (int32 device tensor) makes it per sequence."""
    _require_cuda(q, k_cache, v_cache)
    B, Hq, D = q.shape[0], q.shape[1], q.shape[-1]
    q3 = q[:, :, 0, :] if q.dim() == 4 else q
    max_len = int(kv_len if kv_len is not None else k_cache.shape[2])
    out = torch.empty((B, Hq, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, Hq), dtype=torch.float32, device=q.device)
    L = _lib.load()
    nbytes = L.tyr_b200_attn_decode_workspace_bytes(B, Hq, D, max_len, max_splits)
    if workspace is None:
        workspace = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=q.device)
    a = DecodeArgs()
    a.q, a.o, a.lse = q3.data_ptr(), out.data_ptr(), lse.data_ptr()
    a.k, a.v = k_cache.data_ptr(), v_cache.data_ptr()
    a.k_ptrs = a.v_ptrs = a.kv_head_strides = None
    a.kv_lens = kv_lens.data_ptr() if kv_lens is not None else None
    a.batch, a.n_head, a.n_kv_head, a.max_kv_seq, a.head_dim = B, Hq, k_cache.shape[1], max_len, D
    a.q_stride[:] = [q3.stride(0), q3.stride(1)]
    a.o_stride[:] = [out.stride(0), out.stride(1)]
    a.k_stride[:] = [k_cache.stride(0), k_cache.stride(1), k_cache.stride(2)]
    a.v_stride[:] = [v_cache.stride(0), v_cache.stride(1), v_cache.stride(2)]
    a.scale, a.max_splits = float(scale or 0.0), max_splits
    a.total_kv_len = 0                     # a shared length is known as it is; per-sequence lengths live on the device
    a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel()
    with torch.cuda.device(q.device):
        check(L.tyr_b200_attn_decode(ctypes.byref(a), _stream_ptr(q)))
    return out, lse


def qkPrologue(x: torch.Tensor, out: torch.Tensor, norm_weight: Optional[torch.Tensor] = None,
               cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None,
               positions: Optional[torch.Tensor] = None, position0: int = 0, eps: float = 1e-6,
               pe: Optional[torch.Tensor] = None, out_at_row0: bool = False):
    """Fused per-head RMSNorm + rotary embedding + [B,S,H,D] -> [B,H,S,D] layout change,
    written into `out` [B,H,cap,D] at rows positions[b] + s (in place: a KV-cache append
    when `out` is the cache).  One pass instead of applyHeadNorm
    (Tyr/Model/Qwen/Attention.lean:73-98), rotary.applyRotaryEmb (Tyr/Torch.lean:1043-1048),
    transpose_for_attention (Tyr/Torch.lean:589-597) and data.sliceScatter
    (Tyr/Model/Qwen/Attention.lean:189-193).  `norm_weight` [D] and `cos`/`sin`
    [max_pos, D/2] are float32 device tensors; `positions` is int32 [B].
    `pe` selects Flux's rotary form instead (flux.applyRope, Tyr/Model/Flux/RoPE.lean:71-96): a
    float32 [B or 1, max_pos, D/2, 2, 2] table of 2x2 matrices applied to interleaved pairs
    (the reference's [B, 1, S, D/2, 2, 2] `pe` with its singleton axis dropped).
    `out_at_row0`: the position selects the rotary row only and the result goes to rows 0..S-1 of
    `out` (the query of a decode step: rotated at each sequence's position, stored as row 0).
    Rows that would fall outside `out` or outside the rotary table are refused here when the
    position is known on the host (position0); with device-side `positions` the kernel skips
    them and sets the out-of-range bit of the device status word.
    """
    _require_cuda(x, out)
    if x.dim() != 4 or out.dim() != 4 or x.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise ValueError("x must be bf16 [B,S,H,D] and out bf16 [B,H,cap,D]")
    B, S, H, D = x.shape
    if out.shape[0] != B or out.shape[1] != H or out.shape[3] != D:
        raise ValueError("out does not match x")
    for t_ in (norm_weight, cos, sin, pe):
        if t_ is not None and (t_.dtype != torch.float32 or not t_.is_contiguous() or not t_.is_cuda):
            raise ValueError("norm_weight / cos / sin / pe must be contiguous float32 CUDA tensors")
    if pe is not None:
        if cos is not None or sin is not None:
            raise ValueError("pass either cos/sin or pe")
        if pe.dim() != 5 or tuple(pe.shape[2:]) != (D // 2, 2, 2) or pe.shape[0] not in (1, B):
            raise ValueError("pe must be [B or 1, max_pos, D/2, 2, 2]")
    cap = out.shape[2]
    max_pos = pe.shape[1] if pe is not None else (cos.shape[0] if cos is not None else 0)
    if cos is not None and (sin is None or tuple(cos.shape) != tuple(sin.shape) or cos.dim() != 2 or cos.shape[1] != D // 2):
        raise ValueError("cos and sin must both be [max_pos, D/2]")
    if out_at_row0 and S > cap:
        raise ValueError(f"{S} rows do not fit the {cap} rows of out")
    if positions is None:
        if position0 < 0 or (not out_at_row0 and position0 + S > cap):
            raise ValueError(f"rows {position0}..{position0 + S - 1} do not fit the {cap} rows of out")
        if max_pos and position0 + S > max_pos:
            raise ValueError(f"positions up to {position0 + S - 1} exceed the {max_pos} rows of the rotary table")
    if positions is not None and (positions.dtype != torch.int32 or not positions.is_cuda):
        raise ValueError("positions must be an int32 CUDA tensor")
    a = PrologueArgs()
    a.x, a.out = x.data_ptr(), out.data_ptr()
    a.norm_weight = norm_weight.data_ptr() if norm_weight is not None else None
    a.cos = cos.data_ptr() if cos is not None else None
    a.sin = sin.data_ptr() if sin is not None else None
    a.positions = positions.data_ptr() if positions is not None else None
    a.position0, a.batch, a.seq, a.n_head, a.head_dim = int(position0), B, S, H, D
    a.x_stride[:] = [x.stride(0), x.stride(1), x.stride(2)]
    a.out_stride[:] = [out.stride(0), out.stride(1), out.stride(2)]
    a.eps = float(eps)
    a.cap, a.max_pos, a.out_at_row0 = int(cap), int(max_pos), int(bool(out_at_row0))
    a.pe = pe.data_ptr() if pe is not None else None
    a.pe_batch_stride = pe.stride(0) if (pe is not None and pe.shape[0] > 1) else 0
    with torch.cuda.device(x.device):
        check(_lib.load().tyr_b200_attn_qk_prologue(ctypes.byref(a), _stream_ptr(x)))
    return out


def mergePartials(o_a, lse_a, o_b, lse_b):
    """LSE merge of two partial results (Tyr/GPU/Kernels/RingAttn.lean:164-180)."""
    _require_cuda(o_a, o_b, lse_a, lse_b)
    o_a, o_b = o_a.contiguous().float(), o_b.contiguous().float()
    lse_a, lse_b = lse_a.contiguous().float(), lse_b.contiguous().float()
    out, lse = torch.empty_like(o_a), torch.empty_like(lse_a)
    with torch.cuda.device(o_a.device):
        check(_lib.load().tyr_b200_attn_merge(o_a.data_ptr(), lse_a.data_ptr(), o_b.data_ptr(),
                                              lse_b.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                              lse_a.numel(), o_a.shape[-1], _stream_ptr(o_a)))
    return out, lse


def device_status(device: int = 0, clear: bool = True) -> int:
    """Status word written by the kernels' bounded waits (0 = none gave up)."""
    return int(_lib.load().tyr_b200_attn_device_status(device, int(clear)))


def device_check(device: int = 0) -> None:
    """Raise AttnError if a bounded in-kernel wait gave up or a device-side position or length
    was out of range since the last check; clears the status word."""
    check(int(_lib.load().tyr_b200_attn_device_check(device)))


def launch_count() -> int:
    return int(_lib.load().tyr_b200_attn_launch_count())
