"""The C-ABI library loads and exports what include/tyr_b200_attn.h declares (no GPU, no compute)."""
import ctypes
import os
import re

import pytest

from tyr_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "tyr_b200_attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tyr_b200_\w+)\s*\(", text)))


def test_header_and_binding_list_the_same_symbols():
    assert declared_functions() == sorted(_lib.EXPORTS)


def test_library_exports_every_declared_symbol(built_lib):
    for name in declared_functions():
        assert hasattr(built_lib, name), name


def test_abi_version_and_error_strings(built_lib):
    assert built_lib.tyr_b200_attn_abi_version() == 8
    assert built_lib.tyr_b200_attn_strerror(0) == b"ok"
    for code in range(1, 12):
        assert built_lib.tyr_b200_attn_strerror(-code).startswith(b"tyr_b200_attn:")


def test_struct_sizes_match_the_c_layout():
    # 5 pointers, 6 int32, 12 int64, int32 int32 float int32 int32 (+4 padding), pointer, int64, pointer, int64
    assert ctypes.sizeof(_lib.PrefillArgs) == 5 * 8 + 6 * 4 + 12 * 8 + 5 * 4 + 4 + 8 + 8 + 8 + 8
    assert ctypes.sizeof(_lib.DecodeArgs) == 9 * 8 + 5 * 4 + 4 + 10 * 8 + 4 + 4 + 8 + 8 + 8
    # 10 pointers, uint64, 6 int32, 24 int64, int32 int32 float int32, pointer, int64
    assert ctypes.sizeof(_lib.BackwardArgs) == 10 * 8 + 8 + 6 * 4 + 24 * 8 + 4 * 4 + 8 + 8
    # 6 pointers, 5 int32 (+4 padding), 6 int64, float int32 int32 (+4 padding), pointer, int64, int32 (+4)
    assert ctypes.sizeof(_lib.PrologueArgs) == 6 * 8 + 5 * 4 + 4 + 6 * 8 + 3 * 4 + 4 + 8 + 8 + 4 + 4


def test_arguments_are_rejected_before_any_launch(built_lib):
    a = _lib.PrefillArgs()
    assert built_lib.tyr_b200_attn_prefill(ctypes.byref(a), None) == -1          # NULL pointers
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.addressof(buf)
    p += (-p) % 16
    a.q = a.k = a.v = a.o = p
    a.batch, a.n_head, a.n_kv_head, a.q_seq, a.kv_seq, a.head_dim = 1, 3, 2, 4, 4, 64
    assert built_lib.tyr_b200_attn_prefill(ctypes.byref(a), None) == -2          # 3 % 2 != 0
    a.n_head = 4
    a.head_dim = 96
    assert built_lib.tyr_b200_attn_prefill(ctypes.byref(a), None) == -3          # head_dim
    a.head_dim = 64
    a.dtype = _lib.TYR_ATTN_F32
    assert built_lib.tyr_b200_attn_prefill(ctypes.byref(a), None) == -5          # fp32 outside check mode
    a.dtype = _lib.TYR_ATTN_BF16
    a.q = p + 2
    assert built_lib.tyr_b200_attn_prefill(ctypes.byref(a), None) == -4          # alignment
    # dropout is refused: a Tyr build keeps its LibTorch call for it
    assert built_lib.tyr_b200_sdpa_4d(1, 1, 4, 64, p, p, p, p, 0.1, 1, None) == -6
    assert built_lib.tyr_b200_sdpa_gqa(1, 4, 2, 4, 64, p, p, p, p, 0.0, 1, 0, None) == -2  # enable_gqa off
    # a sliding window needs one sequence length, as the reference's windowed call has
    a.q = p
    for name in ("q_stride", "k_stride", "v_stride", "o_stride"):
        getattr(a, name)[:] = [4 * 8 * 64, 8 * 64, 64]
    a.q_seq, a.kv_seq, a.window_size = 8, 4, 2
    assert built_lib.tyr_b200_attn_prefill(ctypes.byref(a), None) == -2
    a.window_size = -1
    assert built_lib.tyr_b200_attn_prefill(ctypes.byref(a), None) == -2
    d = _lib.DecodeArgs()
    assert built_lib.tyr_b200_attn_decode(ctypes.byref(d), None) == -1
    assert built_lib.tyr_b200_attn_merge(None, None, None, None, None, None, 1, 64, None) == -1


def test_zero_extents_follow_aten(built_lib):
    # an output without elements: nothing to do, NULL pointers allowed
    a = _lib.PrefillArgs()
    a.batch, a.n_head, a.n_kv_head, a.q_seq, a.kv_seq, a.head_dim = 0, 4, 2, 16, 16, 64
    assert built_lib.tyr_b200_attn_prefill(ctypes.byref(a), None) == 0
    a.batch, a.q_seq = 2, 0
    assert built_lib.tyr_b200_attn_prefill(ctypes.byref(a), None) == 0
    assert built_lib.tyr_b200_attn_prefill_host(ctypes.byref(a), 0) == 0
    a.q_seq, a.kv_seq = -1, 0
    assert built_lib.tyr_b200_attn_prefill(ctypes.byref(a), None) == -1         # a negative extent is still refused
    d = _lib.DecodeArgs()
    d.n_head, d.n_kv_head, d.head_dim = 4, 2, 64
    assert built_lib.tyr_b200_attn_decode(ctypes.byref(d), None) == 0           # no sequence
    g = _lib.BackwardArgs()                                                      # gradients of an empty batch: nothing to write
    g.n_head, g.n_kv_head, g.q_seq, g.kv_seq, g.head_dim = 4, 2, 16, 16, 64
    assert built_lib.tyr_b200_attn_backward(ctypes.byref(g), None) == 0
    g.batch, g.q_seq, g.kv_seq = 2, 0, 0                                         # neither queries nor keys
    assert built_lib.tyr_b200_attn_backward(ctypes.byref(g), None) == 0
    g.q_seq = 16                                                                 # no keys: dQ = 0 needs its pointer
    assert built_lib.tyr_b200_attn_backward(ctypes.byref(g), None) == -1
    # no keys: the host-buffer call writes O = 0 and LSE = -inf itself, as ATen's operator returns them
    import numpy as np
    import torch
    B, H, S, D = 2, 4, 3, 64
    o = np.full((B, H, S, D), 0x7fc0, dtype=np.uint16)                             # bf16 NaN bits
    lse = np.zeros((B, H, S), dtype=np.float32)
    a = _lib.PrefillArgs()
    a.o, a.lse = o.ctypes.data, lse.ctypes.data
    a.batch, a.n_head, a.n_kv_head, a.q_seq, a.kv_seq, a.head_dim = B, H, 2, S, 0, D
    a.o_stride[:] = [H * S * D, S * D, D]
    a.dtype = _lib.TYR_ATTN_BF16
    assert built_lib.tyr_b200_attn_prefill_host(ctypes.byref(a), 0) == 0
    assert not o.any() and np.isneginf(lse).all()
    ref = torch.nn.functional.scaled_dot_product_attention(torch.randn(B, H, S, D), torch.randn(B, H, 0, D),
                                                           torch.randn(B, H, 0, D))
    assert not ref.any()


def test_host_call_refuses_strided_tensors(built_lib):
    buf = ctypes.create_string_buffer(1 << 16)
    p = ctypes.addressof(buf)
    a = _lib.PrefillArgs()
    a.q = a.k = a.v = a.o = p
    a.batch, a.n_head, a.n_kv_head, a.q_seq, a.kv_seq, a.head_dim = 2, 2, 2, 4, 4, 64
    a.dtype = _lib.TYR_ATTN_BF16
    for name in ("q_stride", "k_stride", "v_stride", "o_stride"):
        getattr(a, name)[:] = [2 * 4 * 64, 4 * 64, 64]
    a.o_stride[:] = [2 * 4 * 64, 64, 2 * 64]                                     # a [batch, seq, heads, dim] view
    assert built_lib.tyr_b200_attn_prefill_host(ctypes.byref(a), 0) == -2
    a.o_stride[:] = [2 * 4 * 64, 4 * 64, 64]
    a.k_stride[:] = [2 * 8 * 64, 8 * 64, 64]                                     # a window of a longer cache
    assert built_lib.tyr_b200_attn_prefill_host(ctypes.byref(a), 0) == -2
    assert built_lib.tyr_b200_attn_prefill_host(ctypes.byref(a), 64) == -8       # device index out of range


def test_prologue_limits_are_checked_on_the_host(built_lib):
    a = _lib.PrologueArgs()
    assert built_lib.tyr_b200_attn_qk_prologue(ctypes.byref(a), None) == -1     # NULL pointers
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.addressof(buf)
    p += (-p) % 16
    a.x = a.out = p
    a.batch, a.seq, a.n_head, a.head_dim, a.position0 = 1, 4, 2, 64, 0
    a.x_stride[:] = [4 * 2 * 64, 2 * 64, 64]
    a.out_stride[:] = [2 * 8 * 64, 8 * 64, 64]
    assert built_lib.tyr_b200_attn_qk_prologue(ctypes.byref(a), None) == -2     # cap not given
    a.cap, a.position0 = 8, 5
    assert built_lib.tyr_b200_attn_qk_prologue(ctypes.byref(a), None) == -11    # rows 5..8 of an 8-row cache
    a.position0 = 2
    a.cos = a.sin = p
    assert built_lib.tyr_b200_attn_qk_prologue(ctypes.byref(a), None) == -2     # rotary table without max_pos
    a.max_pos = 5
    assert built_lib.tyr_b200_attn_qk_prologue(ctypes.byref(a), None) == -11    # positions 2..5 of a 5-row table
    a.pe = p
    assert built_lib.tyr_b200_attn_qk_prologue(ctypes.byref(a), None) == -2     # two rotary forms at once
    # the test hook refuses limits it cannot honour
    assert built_lib.tyr_b200_attn_test_stalled_wait(0, None) == -2


def test_backward_arguments_and_workspace(built_lib):
    f = built_lib.tyr_b200_attn_backward_workspace_bytes
    assert f(8, 16, 2048) == 2 * 8 * 16 * 2048 * 4
    assert f(1, 2, 100) == 2 * 1 * 2 * 128 * 4              # rows padded to whole 128-row tiles
    assert f(0, 2, 100) == 0
    a = _lib.BackwardArgs()
    assert built_lib.tyr_b200_attn_backward(ctypes.byref(a), None) == -1          # NULL pointers
    buf = ctypes.create_string_buffer(8192)
    p = ctypes.addressof(buf)
    p += (-p) % 16
    a.q = a.k = a.v = a.o = a.d_o = a.lse = a.d_q = a.d_k = a.d_v = p
    a.batch, a.n_head, a.n_kv_head, a.q_seq, a.kv_seq, a.head_dim = 1, 3, 2, 4, 4, 64
    assert built_lib.tyr_b200_attn_backward(ctypes.byref(a), None) == -2          # 3 % 2 != 0
    a.n_head = 4
    a.head_dim = 96
    assert built_lib.tyr_b200_attn_backward(ctypes.byref(a), None) == -3          # head_dim
    a.head_dim = 64
    for name in ("q_stride", "k_stride", "v_stride", "o_stride", "do_stride", "dq_stride", "dk_stride", "dv_stride"):
        getattr(a, name)[:] = [4 * 4 * 64, 4 * 64, 64]
    assert built_lib.tyr_b200_attn_backward(ctypes.byref(a), None) == -7          # no workspace
    a.workspace, a.workspace_bytes = p, 16
    assert built_lib.tyr_b200_attn_backward(ctypes.byref(a), None) == -7          # workspace too small
    a.dtype = _lib.TYR_ATTN_F32
    assert built_lib.tyr_b200_attn_backward(ctypes.byref(a), None) == -5          # bf16 only


def test_decode_workspace_formula(built_lib):
    f = built_lib.tyr_b200_attn_decode_workspace_bytes
    assert f(64, 32, 128, 200, 64) == 0                      # one chunk: no scratch
    assert f(64, 32, 128, 32768, 64) == 64 * 32 * 64 * 129 * 4
    assert f(1, 8, 64, 1000, 64) == 1 * 8 * 4 * 65 * 4       # 256-key chunks -> 4 splits


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError):
        _lib.load()
