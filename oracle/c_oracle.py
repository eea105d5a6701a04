"""ctypes binding of attn_oracle.c (numpy in, numpy out).  Test infrastructure only."""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libattn_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "attn_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libattn_oracle.so"], stdout=subprocess.DEVNULL)
    return _SO


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_SO)
        f32p = ctypes.POINTER(ctypes.c_float)
        L.tyr_oracle_sdpa.argtypes = [f32p, f32p, f32p, f32p, f32p] + [ctypes.c_int] * 7 + [ctypes.c_float]
        L.tyr_oracle_sdpa.restype = ctypes.c_int
        L.tyr_oracle_sdpa_window.argtypes = [f32p, f32p, f32p, f32p, f32p] + [ctypes.c_int] * 5 + [ctypes.c_float, ctypes.c_int]
        L.tyr_oracle_sdpa_window.restype = ctypes.c_int
        L.tyr_oracle_sdpa_keymask.argtypes = [f32p, f32p, f32p, f32p, f32p] + [ctypes.c_int] * 6 + [ctypes.c_float, ctypes.POINTER(ctypes.c_uint8)]
        L.tyr_oracle_sdpa_keymask.restype = ctypes.c_int
        L.tyr_oracle_sdpa_online.argtypes = (
            [f32p, f32p, f32p, f32p, f32p] + [ctypes.c_int] * 7 + [ctypes.c_float, ctypes.c_int]
        )
        L.tyr_oracle_sdpa_online.restype = ctypes.c_int
        L.tyr_oracle_sdpa_backward.argtypes = [f32p] * 7 + [ctypes.c_int] * 7 + [ctypes.c_float]
        L.tyr_oracle_sdpa_backward.restype = ctypes.c_int
        L.tyr_oracle_sdpa_backward_masked.argtypes = ([f32p] * 7 + [ctypes.c_int] * 7 + [ctypes.c_float, ctypes.c_int,
                                                      ctypes.POINTER(ctypes.c_uint8)])
        L.tyr_oracle_sdpa_backward_masked.restype = ctypes.c_int
        L.tyr_oracle_merge2.argtypes = [f32p] * 6 + [ctypes.c_int64, ctypes.c_int]
        L.tyr_oracle_merge2.restype = None
        L.tyr_oracle_bf16_round.argtypes = [f32p, f32p, ctypes.c_int64]
        L.tyr_oracle_bf16_round.restype = None
        i32p = ctypes.POINTER(ctypes.c_int32)
        L.tyr_oracle_qk_prologue.argtypes = [f32p, f32p, f32p, f32p, i32p, ctypes.c_int, f32p] + [ctypes.c_int] * 5 + [ctypes.c_float]
        L.tyr_oracle_qk_prologue.restype = None
        L.tyr_oracle_qk_prologue_pe.argtypes = [f32p, f32p, f32p, ctypes.c_int64, i32p, ctypes.c_int, f32p] + [ctypes.c_int] * 5 + [ctypes.c_float]
        L.tyr_oracle_qk_prologue_pe.restype = None
        L.tyr_oracle_threads.restype = ctypes.c_int
        L.tyr_oracle_set_threads.argtypes = [ctypes.c_int]
        _lib = L
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def _c(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32))


def threads() -> int:
    return int(lib().tyr_oracle_threads())


def sdpa_backward(q, k, v, d_o, is_causal: bool, scale: float | None = None, window: int = 0, key_mask=None):
    """Gradients of `sdpa` for the cotangent d_o: (d_q [B,Hq,Sq,D], d_k, d_v [B,Hkv,Skv,D]).
    `window` / `key_mask` as in `sdpa`."""
    q, k, v, d_o = _c(q), _c(k), _c(v), _c(d_o)
    B, Hq, Sq, D = q.shape
    _, Hkv, Skv, _ = k.shape
    assert k.shape == v.shape and k.shape[0] == B and k.shape[3] == D and d_o.shape == q.shape
    if scale is None:
        scale = 1.0 / float(np.sqrt(D))
    d_q, d_k, d_v = np.empty_like(q), np.empty_like(k), np.empty_like(v)
    if window or key_mask is not None:
        km = None
        if key_mask is not None:
            km = np.ascontiguousarray(np.asarray(key_mask) != 0, dtype=np.uint8)
            assert km.shape == (B, Skv)
        rc = lib().tyr_oracle_sdpa_backward_masked(
            _p(q), _p(k), _p(v), _p(d_o), _p(d_q), _p(d_k), _p(d_v), B, Hq, Hkv, Sq, Skv, D, int(bool(is_causal)),
            scale, int(window), km.ctypes.data_as(ctypes.POINTER(ctypes.c_uint8)) if km is not None else None)
    else:
        rc = lib().tyr_oracle_sdpa_backward(_p(q), _p(k), _p(v), _p(d_o), _p(d_q), _p(d_k), _p(d_v), B, Hq, Hkv,
                                            Sq, Skv, D, int(bool(is_causal)), scale)
    if rc != 0:
        raise ValueError("tyr_oracle_sdpa_backward rejected its arguments")
    return d_q, d_k, d_v


def sdpa(q, k, v, is_causal: bool, scale: float | None = None, online_block: int = 0, window: int = 0,
         key_mask=None):
    """q [B,Hq,Sq,D], k/v [B,Hkv,Skv,D] fp32 -> (o [B,Hq,Sq,D], lse [B,Hq,Sq])."""
    q, k, v = _c(q), _c(k), _c(v)
    B, Hq, Sq, D = q.shape
    _, Hkv, Skv, _ = k.shape
    assert k.shape == v.shape and k.shape[0] == B and k.shape[3] == D
    if scale is None:
        scale = 1.0 / float(np.sqrt(D))
    o = np.empty_like(q)
    lse = np.empty((B, Hq, Sq), dtype=np.float32)
    if key_mask is not None:
        assert Sq == Skv and not window
        km = np.ascontiguousarray(np.asarray(key_mask) != 0, dtype=np.uint8)
        assert km.shape == (B, Skv)
        rc = lib().tyr_oracle_sdpa_keymask(_p(q), _p(k), _p(v), _p(o), _p(lse), B, Hq, Hkv, Sq, D,
                                           int(bool(is_causal)), scale,
                                           km.ctypes.data_as(ctypes.POINTER(ctypes.c_uint8)))
    elif window:
        assert Sq == Skv
        rc = lib().tyr_oracle_sdpa_window(_p(q), _p(k), _p(v), _p(o), _p(lse), B, Hq, Hkv, Sq, D, scale, int(window))
    elif online_block:
        rc = lib().tyr_oracle_sdpa_online(_p(q), _p(k), _p(v), _p(o), _p(lse), B, Hq, Hkv, Sq, Skv, D,
                                          int(bool(is_causal)), scale, online_block)
    else:
        rc = lib().tyr_oracle_sdpa(_p(q), _p(k), _p(v), _p(o), _p(lse), B, Hq, Hkv, Sq, Skv, D,
                                   int(bool(is_causal)), scale)
    if rc != 0:
        raise ValueError("tyr_oracle_sdpa rejected its arguments")
    return o, lse


def merge2(o_a, lse_a, o_b, lse_b):
    o_a, o_b, lse_a, lse_b = _c(o_a), _c(o_b), _c(lse_a), _c(lse_b)
    rows, D = lse_a.size, o_a.shape[-1]
    o = np.empty_like(o_a)
    lse = np.empty_like(lse_a)
    lib().tyr_oracle_merge2(_p(o_a), _p(lse_a), _p(o_b), _p(lse_b), _p(o), _p(lse), rows, D)
    return o, lse


def bf16_round(x) -> np.ndarray:
    x = _c(x)
    out = np.empty_like(x)
    lib().tyr_oracle_bf16_round(_p(x), _p(out), x.size)
    return out


def qk_prologue(x, out, weight=None, cos=None, sin=None, positions=None, position0=0, eps=1e-6):
    """x [B,S,H,D] fp32; out [B,H,cap,D] fp32 is updated in place and returned."""
    x = _c(x)
    assert out.dtype == np.float32 and out.flags["C_CONTIGUOUS"]
    B, S, H, D = x.shape
    cap = out.shape[2]
    null = ctypes.POINTER(ctypes.c_float)()
    w = _c(weight) if weight is not None else None
    cs = _c(cos) if cos is not None else None
    sn = _c(sin) if sin is not None else None
    pos = np.ascontiguousarray(positions, dtype=np.int32) if positions is not None else None
    lib().tyr_oracle_qk_prologue(
        _p(x), _p(w) if w is not None else null, _p(cs) if cs is not None else null,
        _p(sn) if sn is not None else null,
        pos.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)) if pos is not None else ctypes.POINTER(ctypes.c_int32)(),
        int(position0), _p(out), B, S, H, D, cap, float(eps))
    return out


def qk_prologue_pe(x, out, pe, weight=None, positions=None, position0=0, eps=1e-6):
    """`qk_prologue` with Flux's interleaved-pair rotary: pe [B or 1, max_pos, D/2, 2, 2] fp32."""
    x, pe = _c(x), _c(pe)
    assert out.dtype == np.float32 and out.flags["C_CONTIGUOUS"]
    B, S, H, D = x.shape
    cap = out.shape[2]
    assert pe.shape[2:] == (D // 2, 2, 2) and pe.shape[0] in (1, B)
    stride = 0 if pe.shape[0] == 1 else pe.shape[1] * 2 * D
    w = _c(weight) if weight is not None else None
    pos = np.ascontiguousarray(positions, dtype=np.int32) if positions is not None else None
    lib().tyr_oracle_qk_prologue_pe(
        _p(x), _p(w) if w is not None else ctypes.POINTER(ctypes.c_float)(), _p(pe), stride,
        pos.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)) if pos is not None else ctypes.POINTER(ctypes.c_int32)(),
        int(position0), _p(out), B, S, H, D, cap, float(eps))
    return out
