"""ctypes binding of the C ABI declared in include/tyr_b200_attn.h.

There is no fallback: if the shared library is missing the import of any
operator raises, it never routes to PyTorch or to a CPU path.
"""
from __future__ import annotations

import ctypes
import os

from .build import LIB_PATH

c_i32, c_i64, c_u64, c_f32, c_f64, c_u8 = (ctypes.c_int32, ctypes.c_int64, ctypes.c_uint64,
                                           ctypes.c_float, ctypes.c_double, ctypes.c_uint8)
vp = ctypes.c_void_p

TYR_ATTN_BF16, TYR_ATTN_F32 = 0, 1
DECODE_STATIC_SCRATCH_BYTES = 16 << 20   # TYR_ATTN_DECODE_STATIC_SCRATCH_BYTES

# every symbol include/tyr_b200_attn.h declares
EXPORTS = [
    "tyr_b200_attn_prefill", "tyr_b200_attn_prefill_workspace_bytes", "tyr_b200_sdpa_4d", "tyr_b200_sdpa_gqa", "tyr_b200_sdpa_gqa_qkv",
    "tyr_b200_sdpa_gqa_window", "tyr_b200_sdpa_gqa_mask",
    "tyr_b200_attn_decode_workspace_bytes", "tyr_b200_attn_decode", "tyr_b200_attn_decode_static",
    "tyr_b200_attn_merge", "tyr_b200_attn_qk_prologue",
    "tyr_b200_attn_backward_workspace_bytes", "tyr_b200_attn_backward",
    "tyr_b200_attn_prefill_host", "tyr_b200_attn_device_status", "tyr_b200_attn_device_check",
    "tyr_b200_attn_test_set_wait_limit", "tyr_b200_attn_test_stalled_wait", "tyr_b200_attn_strerror",
    "tyr_b200_attn_abi_version", "tyr_b200_attn_launch_count",
]


class PrefillArgs(ctypes.Structure):
    _fields_ = [
        ("q", vp), ("k", vp), ("v", vp), ("o", vp), ("lse", vp),
        ("batch", c_i32), ("n_head", c_i32), ("n_kv_head", c_i32), ("q_seq", c_i32),
        ("kv_seq", c_i32), ("head_dim", c_i32),
        ("q_stride", c_i64 * 3), ("k_stride", c_i64 * 3), ("v_stride", c_i64 * 3),
        ("o_stride", c_i64 * 3),
        ("dtype", c_i32), ("is_causal", c_i32), ("scale", c_f32), ("check_mode", c_i32),
        ("window_size", c_i32), ("key_mask", vp), ("key_mask_stride", c_i64),
        ("workspace", vp), ("workspace_bytes", c_i64),
    ]


class DecodeArgs(ctypes.Structure):
    _fields_ = [
        ("q", vp), ("o", vp), ("lse", vp), ("k", vp), ("v", vp),
        ("k_ptrs", vp), ("v_ptrs", vp), ("kv_lens", vp), ("kv_head_strides", vp),
        ("batch", c_i32), ("n_head", c_i32), ("n_kv_head", c_i32), ("max_kv_seq", c_i32),
        ("head_dim", c_i32),
        ("q_stride", c_i64 * 2), ("o_stride", c_i64 * 2), ("k_stride", c_i64 * 3),
        ("v_stride", c_i64 * 3),
        ("scale", c_f32), ("max_splits", c_i32), ("workspace", vp), ("workspace_bytes", ctypes.c_size_t),
        ("total_kv_len", c_i64),
    ]


class PrologueArgs(ctypes.Structure):
    _fields_ = [
        ("x", vp), ("out", vp), ("norm_weight", vp), ("cos", vp), ("sin", vp), ("positions", vp),
        ("position0", c_i32), ("batch", c_i32), ("seq", c_i32), ("n_head", c_i32), ("head_dim", c_i32),
        ("x_stride", c_i64 * 3), ("out_stride", c_i64 * 3), ("eps", c_f32),
        ("cap", c_i32), ("max_pos", c_i32), ("pe", vp), ("pe_batch_stride", c_i64), ("out_at_row0", c_i32),
    ]


class BackwardArgs(ctypes.Structure):
    _fields_ = [
        ("q", vp), ("k", vp), ("v", vp), ("o", vp), ("d_o", vp), ("lse", vp),
        ("d_q", vp), ("d_k", vp), ("d_v", vp), ("workspace", vp), ("workspace_bytes", c_u64),
        ("batch", c_i32), ("n_head", c_i32), ("n_kv_head", c_i32), ("q_seq", c_i32),
        ("kv_seq", c_i32), ("head_dim", c_i32),
        ("q_stride", c_i64 * 3), ("k_stride", c_i64 * 3), ("v_stride", c_i64 * 3),
        ("o_stride", c_i64 * 3), ("do_stride", c_i64 * 3),
        ("dq_stride", c_i64 * 3), ("dk_stride", c_i64 * 3), ("dv_stride", c_i64 * 3),
        ("dtype", c_i32), ("is_causal", c_i32), ("scale", c_f32),
        ("window_size", c_i32), ("key_mask", vp), ("key_mask_stride", c_i64),
    ]


_lib = None


def load() -> ctypes.CDLL:
    """Load lib/libtyr_b200_attn.so; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: run `python -c 'import __graft_entry__ as g; g.build()'` "
            "(or tyr_b200.build.build()).  There is no CPU or PyTorch fallback.")
    L = ctypes.CDLL(LIB_PATH)
    L.tyr_b200_attn_prefill.argtypes = [ctypes.POINTER(PrefillArgs), vp]
    L.tyr_b200_attn_prefill.restype = ctypes.c_int
    L.tyr_b200_attn_prefill_host.argtypes = [ctypes.POINTER(PrefillArgs), c_i32]
    L.tyr_b200_attn_prefill_host.restype = ctypes.c_int
    L.tyr_b200_sdpa_4d.argtypes = [c_u64] * 4 + [vp] * 4 + [c_f64, c_u8, vp]
    L.tyr_b200_sdpa_4d.restype = ctypes.c_int
    L.tyr_b200_sdpa_gqa.argtypes = [c_u64] * 5 + [vp] * 4 + [c_f64, c_u8, c_u8, vp]
    L.tyr_b200_sdpa_gqa.restype = ctypes.c_int
    L.tyr_b200_sdpa_gqa_qkv.argtypes = [c_u64] * 6 + [vp] * 4 + [c_f64, c_u8, c_u8, vp]
    L.tyr_b200_sdpa_gqa_qkv.restype = ctypes.c_int
    L.tyr_b200_sdpa_gqa_window.argtypes = [c_u64] * 5 + [vp] * 4 + [c_f64, c_u8, c_u8, c_u64, vp]
    L.tyr_b200_sdpa_gqa_window.restype = ctypes.c_int
    L.tyr_b200_sdpa_gqa_mask.argtypes = [c_u64] * 5 + [vp] * 5 + [c_f64, c_u8, c_u8, vp]
    L.tyr_b200_sdpa_gqa_mask.restype = ctypes.c_int
    L.tyr_b200_attn_prefill_workspace_bytes.argtypes = [ctypes.POINTER(PrefillArgs)]
    L.tyr_b200_attn_prefill_workspace_bytes.restype = c_i64
    L.tyr_b200_attn_decode_workspace_bytes.argtypes = [c_i32] * 5
    L.tyr_b200_attn_decode_workspace_bytes.restype = ctypes.c_size_t
    L.tyr_b200_attn_decode.argtypes = [ctypes.POINTER(DecodeArgs), vp]
    L.tyr_b200_attn_decode.restype = ctypes.c_int
    L.tyr_b200_attn_decode_static.argtypes = [ctypes.POINTER(DecodeArgs), vp]
    L.tyr_b200_attn_decode_static.restype = ctypes.c_int
    L.tyr_b200_attn_qk_prologue.argtypes = [ctypes.POINTER(PrologueArgs), vp]
    L.tyr_b200_attn_qk_prologue.restype = ctypes.c_int
    L.tyr_b200_attn_backward_workspace_bytes.argtypes = [c_i32] * 3
    L.tyr_b200_attn_backward_workspace_bytes.restype = c_u64
    L.tyr_b200_attn_backward.argtypes = [ctypes.POINTER(BackwardArgs), vp]
    L.tyr_b200_attn_backward.restype = ctypes.c_int
    L.tyr_b200_attn_merge.argtypes = [vp] * 6 + [c_i64, c_i32, vp]
    L.tyr_b200_attn_merge.restype = ctypes.c_int
    L.tyr_b200_attn_device_status.argtypes = [c_i32, c_i32]
    L.tyr_b200_attn_device_status.restype = ctypes.c_int
    L.tyr_b200_attn_device_check.argtypes = [c_i32]
    L.tyr_b200_attn_device_check.restype = ctypes.c_int
    L.tyr_b200_attn_test_set_wait_limit.argtypes = [c_i64]
    L.tyr_b200_attn_test_set_wait_limit.restype = None
    L.tyr_b200_attn_test_stalled_wait.argtypes = [c_i64, vp]
    L.tyr_b200_attn_test_stalled_wait.restype = ctypes.c_int
    L.tyr_b200_attn_strerror.argtypes = [ctypes.c_int]
    L.tyr_b200_attn_strerror.restype = ctypes.c_char_p
    L.tyr_b200_attn_abi_version.restype = ctypes.c_int
    L.tyr_b200_attn_launch_count.restype = c_u64
    _lib = L
    return L


class AttnError(RuntimeError):
    """Raised with the library's own message, like the IO error of Tyr's launchers."""

    def __init__(self, code: int):
        self.code = code
        super().__init__(load().tyr_b200_attn_strerror(code).decode())


def check(code: int) -> None:
    if code != 0:
        raise AttnError(code)
