"""Parity of the backward kernels (through the C ABI) with the oracle and the stored autograd gradients."""
import numpy as np
import pytest
import torch

from conftest import GRAD_REL_TO_MAX
from oracle import c_oracle

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda:0")


def _bf16(a):
    return torch.from_numpy(np.ascontiguousarray(a)).bfloat16().to(_dev())


def _run(q, k, v, d_o, causal, scale=None):
    from tyr_b200 import nn as tnn
    o, lse = tnn.attentionFwd(q, k, v, is_causal=causal, scale=scale)
    d_q, d_k, d_v = tnn.attentionBwd(q, k, v, o, lse, d_o, is_causal=causal, scale=scale)
    torch.cuda.synchronize()
    assert tnn.device_status(0, True) == 0
    return d_q, d_k, d_v


def _close(got, want, what):
    got = got.float().cpu().numpy()
    err = np.abs(got - want).max() / max(np.abs(want).max(), 1e-6)
    assert np.isfinite(got).all(), what
    assert err <= GRAD_REL_TO_MAX, f"{what}: max-abs error {err:.3e} of the largest entry"


def test_golden_autograd_gradients(golden_backward):
    for name, c in golden_backward.items():
        causal = bool(c["meta"][6])
        got = _run(_bf16(c["q"]), _bf16(c["k"]), _bf16(c["v"]), _bf16(c["d_o"]), causal)
        for g, key in zip(got, ("d_q", "d_k", "d_v")):
            _close(g, c[key], f"{name}.{key}")


CASES = [
    # B, Hq, Hkv, Sq, Skv, D, causal
    (1, 1, 1, 128, 128, 128, False),
    (1, 1, 1, 128, 128, 128, True),
    (2, 4, 2, 384, 384, 64, True),
    (1, 2, 2, 200, 333, 128, False),
    (2, 4, 1, 100, 100, 64, True),
    (1, 2, 1, 128, 512, 128, True),      # more keys than queries: the late keys get zero gradient
    (1, 2, 2, 512, 128, 128, True),      # more queries than keys
    (1, 6, 2, 257, 257, 128, True),      # group of three, one row past a tile edge
    (1, 8, 8, 1, 300, 64, False),        # a single query row
    (3, 2, 1, 64, 64, 64, True),
    (1, 4, 2, 2048, 2048, 128, True),    # 16 tiles per side: many units per CTA round, long accumulations
    (1, 2, 2, 1500, 1500, 64, False),
    (160, 1, 1, 130, 130, 64, True),     # more work units than SMs: several rounds of the persistent schedule
]


@pytest.mark.parametrize("B,Hq,Hkv,Sq,Skv,D,causal", CASES)
def test_against_the_oracle(B, Hq, Hkv, Sq, Skv, D, causal):
    g = torch.Generator().manual_seed(B * 1000 + Sq + Skv + D)
    q, k, v, d_o = (torch.randn(s, generator=g).bfloat16() for s in
                    ((B, Hq, Sq, D), (B, Hkv, Skv, D), (B, Hkv, Skv, D), (B, Hq, Sq, D)))
    want = c_oracle.sdpa_backward(q.float().numpy(), k.float().numpy(), v.float().numpy(), d_o.float().numpy(), causal)
    got = _run(q.to(_dev()), k.to(_dev()), v.to(_dev()), d_o.to(_dev()), causal)
    for gt, w, key in zip(got, want, ("d_q", "d_k", "d_v")):
        _close(gt, w, key)


def test_custom_scale_and_strided_inputs():
    """Q/K/V/dO as [B,S,H,D] views (the layout before transpose_for_attention) and a scale that is not 1/sqrt(D)."""
    g = torch.Generator().manual_seed(11)
    B, Hq, Hkv, S, D = 2, 4, 2, 160, 64
    qs, ds = (torch.randn(B, S, Hq, D, generator=g).bfloat16() for _ in range(2))
    ks, vs = (torch.randn(B, S, Hkv, D, generator=g).bfloat16() for _ in range(2))
    q, k, v, d_o = (t.to(_dev()).transpose(1, 2) for t in (qs, ks, vs, ds))
    scale = 0.2
    want = c_oracle.sdpa_backward(*(t.float().cpu().contiguous().numpy() for t in (q, k, v, d_o)), True, scale)
    from tyr_b200 import nn as tnn
    o, lse = tnn.attentionFwd(q, k, v, is_causal=True, scale=scale)
    got = tnn.attentionBwd(q, k, v, o, lse, d_o, is_causal=True, scale=scale)
    torch.cuda.synchronize()
    for gt, w, key in zip(got, want, ("d_q", "d_k", "d_v")):
        _close(gt, w, key)


def test_linearity_in_the_cotangent():
    """Gradients are linear in dO: bwd(2 dO) = 2 bwd(dO) bit for bit (a power of two scales every product exactly)."""
    g = torch.Generator().manual_seed(12)
    q, k, v, d_o = (torch.randn(1, 2, 256, 128, generator=g).bfloat16().to(_dev()) for _ in range(4))
    a = _run(q, k, v, d_o, True)
    b = _run(q, k, v, d_o * 2, True)
    for x, y in zip(a, b):
        assert torch.equal((x.float() * 2).bfloat16(), y)


def test_keys_beyond_every_query_get_zero_gradient():
    g = torch.Generator().manual_seed(13)
    q, d_o = (torch.randn(1, 2, 100, 64, generator=g).bfloat16().to(_dev()) for _ in range(2))
    k, v = (torch.randn(1, 1, 400, 64, generator=g).bfloat16().to(_dev()) for _ in range(2))
    _, d_k, d_v = _run(q, k, v, d_o, True)
    assert torch.count_nonzero(d_k[:, :, 100:]) == 0 and torch.count_nonzero(d_v[:, :, 100:]) == 0


def test_workspace_is_checked_and_reusable():
    from tyr_b200 import nn as tnn, _lib
    g = torch.Generator().manual_seed(14)
    q, k, v, d_o = (torch.randn(1, 2, 130, 64, generator=g).bfloat16().to(_dev()) for _ in range(4))
    o, lse = tnn.attentionFwd(q, k, v)
    need = _lib.load().tyr_b200_attn_backward_workspace_bytes(1, 2, 130)
    assert need == 2 * 2 * 256 * 4
    with pytest.raises(ValueError):
        tnn.attentionBwd(q, k, v, o, lse, d_o, workspace=torch.empty(8, device=_dev()))
    ws = torch.empty(need // 4, device=_dev())
    a = tnn.attentionBwd(q, k, v, o, lse, d_o, workspace=ws)
    b = tnn.attentionBwd(q, k, v, o, lse, d_o, workspace=ws)
    for x, y in zip(a, b):
        assert torch.equal(x, y)


def test_full_headline_shape_properties():
    """Headline shape (B=8, 16/8 heads, S=2048, D=128, causal): exact oracle gradients for one batch element
    are too slow on the CPU here, so this checks size-independent properties on the full launch and the oracle
    on a slice: (1) the batch elements are independent, so the gradients of element 0 equal those of a
    one-element call bit for bit; (2) sum over queries of dQ.q equals sum over keys of dK.k for every KV head
    (both are sum_ij dS_ij S_ij / scale), within accumulation error."""
    from tyr_b200 import nn as tnn
    g = torch.Generator().manual_seed(21)
    B, Hq, Hkv, S, D = 8, 16, 8, 2048, 128
    q, d_o = (torch.randn(B, Hq, S, D, generator=g).bfloat16().to(_dev()) for _ in range(2))
    k, v = (torch.randn(B, Hkv, S, D, generator=g).bfloat16().to(_dev()) for _ in range(2))
    d_q, d_k, d_v = _run(q, k, v, d_o, True)
    one = _run(q[:1], k[:1], v[:1], d_o[:1], True)
    for full, single in zip((d_q, d_k, d_v), one):
        assert torch.equal(full[:1], single)
    lhs = (d_q.float() * q.float()).sum(dim=(2, 3)).view(B, Hkv, Hq // Hkv).sum(-1)
    rhs = (d_k.float() * k.float()).sum(dim=(2, 3))
    scale = (d_q.float().abs() * q.float().abs()).sum(dim=(2, 3)).view(B, Hkv, Hq // Hkv).sum(-1)
    assert ((lhs - rhs).abs() / scale).max().item() < 2e-3


@pytest.mark.parametrize("B,Hq,Hkv,S,D,window", [(1, 2, 1, 200, 64, 7), (2, 2, 2, 400, 128, 140),
                                                 (1, 4, 2, 1000, 128, 300), (1, 1, 1, 130, 64, 2)])
def test_sliding_window_backward(B, Hq, Hkv, S, D, window):
    """Backward of the windowed call (lean_torch_sdpa_gqa_window under autograd) against the oracle."""
    from tyr_b200 import nn as tnn
    g = torch.Generator().manual_seed(S + window)
    q, d_o = (torch.randn(B, Hq, S, D, generator=g).bfloat16() for _ in range(2))
    k, v = (torch.randn(B, Hkv, S, D, generator=g).bfloat16() for _ in range(2))
    want = c_oracle.sdpa_backward(*(t.float().numpy() for t in (q, k, v, d_o)), True, window=window)
    qd, kd, vd, dd = (t.to(_dev()) for t in (q, k, v, d_o))
    o, lse = tnn.attentionFwd(qd, kd, vd, window_size=window)
    got = tnn.attentionBwd(qd, kd, vd, o, lse, dd, window_size=window)
    torch.cuda.synchronize()
    assert tnn.device_status(0, True) == 0
    for gt, w, key in zip(got, want, ("d_q", "d_k", "d_v")):
        _close(gt, w, key)


@pytest.mark.parametrize("causal", [True, False])
def test_padding_mask_backward(causal):
    """Backward of the padding-masked call against the oracle; padding keys get exactly zero gradient."""
    from tyr_b200 import nn as tnn
    g = torch.Generator().manual_seed(41)
    B, Hq, Hkv, S, D = 3, 4, 2, 300, 128
    q, d_o = (torch.randn(B, Hq, S, D, generator=g).bfloat16() for _ in range(2))
    k, v = (torch.randn(B, Hkv, S, D, generator=g).bfloat16() for _ in range(2))
    m = torch.ones(B, S, dtype=torch.uint8)
    m[0, 170:] = 0          # right padding
    m[1, 20:45] = 0         # a hole
    m[1, 128:260] = 0       # a whole tile and more
    want = c_oracle.sdpa_backward(*(t.float().numpy() for t in (q, k, v, d_o)), causal, key_mask=m.numpy())
    qd, kd, vd, dd, md = (t.to(_dev()) for t in (q, k, v, d_o, m))
    o, lse = tnn.attentionFwd(qd, kd, vd, is_causal=causal, key_mask=md)
    got = tnn.attentionBwd(qd, kd, vd, o, lse, dd, is_causal=causal, key_mask=md)
    torch.cuda.synchronize()
    assert tnn.device_status(0, True) == 0
    for gt, w, key in zip(got, want, ("d_q", "d_k", "d_v")):
        _close(gt, w, key)
    assert torch.count_nonzero(got[1][0, :, 170:]) == 0 and torch.count_nonzero(got[2][1, :, 128:260]) == 0


def test_window_of_one_is_closed_form():
    """window_size = 1: every query sees only its own key, P = 1, so dV_j is the sum of the group's dO_j exactly
    and dQ, dK vanish (up to the bf16 rounding of O inside delta)."""
    from tyr_b200 import nn as tnn
    g = torch.Generator().manual_seed(51)
    q, d_o = (torch.randn(1, 2, 130, 64, generator=g).bfloat16().to(_dev()) for _ in range(2))
    k, v = (torch.randn(1, 1, 130, 64, generator=g).bfloat16().to(_dev()) for _ in range(2))
    o, lse = tnn.attentionFwd(q, k, v, window_size=1)
    d_q, d_k, d_v = tnn.attentionBwd(q, k, v, o, lse, d_o, window_size=1)
    torch.cuda.synchronize()
    assert torch.equal(d_v, (d_o[:, 0].float() + d_o[:, 1].float()).bfloat16()[:, None])
    assert d_q.float().abs().max().item() < 0.1 and d_k.float().abs().max().item() < 0.1


def _block_grads_f64(q, k, v, d_o, b, hkv, j0, j1, causal, scale):
    """Exact dK, dV of the key block [j0, j1) of (batch b, KV head hkv) and exact dQ of the query rows
    [j0, j1) of the group's first query head, in float64 with numpy.  The formulas are the backward
    of Tyr/GPU/Kernels/MhaH100.lean:196-344 (the ones tyr_oracle_sdpa_backward implements); only the
    query rows that can see the block enter, so the cost stays bounded at any sequence length.
    q [B,Hq,S,D], k/v [B,Hkv,S,D], d_o like q: float32 numpy arrays (bf16-representable values)."""
    Hq, Hkv, S, D = q.shape[1], k.shape[1], q.shape[2], q.shape[3]
    g = Hq // Hkv
    kk, vv = k[b, hkv].astype(np.float64), v[b, hkv].astype(np.float64)
    i0 = j0 if causal else 0                       # first query row that sees key j0
    d_k = np.zeros((j1 - j0, D)); d_v = np.zeros((j1 - j0, D))
    d_q_first = None
    for h in range(hkv * g, (hkv + 1) * g):
        qq, dd = q[b, h, i0:].astype(np.float64), d_o[b, h, i0:].astype(np.float64)
        s = qq @ kk.T * scale                      # [rows, S]
        if causal:
            rows = np.arange(i0, S)[:, None]
            s = np.where(np.arange(S)[None, :] > rows, -np.inf, s)
        m = s.max(axis=1, keepdims=True)
        p = np.exp(s - m)
        p /= p.sum(axis=1, keepdims=True)
        o = p @ vv
        delta = (dd * o).sum(axis=1, keepdims=True)
        d_s = p * (dd @ vv.T - delta) * scale      # [rows, S]
        d_v += p[:, j0:j1].T @ dd
        d_k += d_s[:, j0:j1].T @ qq
        if h == hkv * g:
            lo = j0 - i0
            d_q_first = d_s[lo:lo + (j1 - j0)] @ kk
    return d_k, d_v, d_q_first


def test_block_formulas_agree_with_the_oracle():
    """The float64 block helper above is pinned to tyr_oracle_sdpa_backward on a small case."""
    rng = np.random.default_rng(3)
    bf = lambda a: torch.from_numpy(a.astype(np.float32)).bfloat16().float().numpy()
    q, k, v, d_o = bf(rng.standard_normal((1, 4, 96, 64))), bf(rng.standard_normal((1, 2, 96, 64))), \
        bf(rng.standard_normal((1, 2, 96, 64))), bf(rng.standard_normal((1, 4, 96, 64)))
    for causal in (True, False):
        w_q, w_k, w_v = c_oracle.sdpa_backward(q, k, v, d_o, causal)
        d_k, d_v, d_q = _block_grads_f64(q, k, v, d_o, 0, 1, 32, 64, causal, 0.125)
        assert np.abs(d_k - w_k[0, 1, 32:64]).max() <= 1e-4
        assert np.abs(d_v - w_v[0, 1, 32:64]).max() <= 1e-4
        assert np.abs(d_q - w_q[0, 2, 32:64]).max() <= 1e-4


@pytest.mark.parametrize("name", ["qwen3_0p6b_prefill", "qwen3_8b_prefill"])
def test_benchmark_shapes_by_sampled_key_blocks_and_rows(name):
    """The backward at the two sizes it is benchmarked on, checked against exact float64 gradients
    of sampled 128-key blocks (dK, dV, summed over the whole GQA group) and 128 query rows (dQ)."""
    from tyr_b200 import nn as tnn
    from tyr_b200 import workloads as W
    w = W.WORKLOADS[name]
    qh, kh, vh = W.make_prefill(w)
    g = torch.Generator(device="cpu").manual_seed(w.seed + 100)
    dh = torch.randn(qh.shape, generator=g).bfloat16()
    q, k, v, d_o = (t.to(_dev()) for t in (qh, kh, vh, dh))
    o, lse = tnn.attentionFwd(q, k, v, is_causal=w.causal)
    d_q, d_k, d_v = tnn.attentionBwd(q, k, v, o, lse, d_o, is_causal=w.causal)
    torch.cuda.synchronize()
    assert tnn.device_status(0, True) == 0
    qn, kn, vn, dn = (t.float().numpy() for t in (qh, kh, vh, dh))
    S = w.seq
    g_ = w.n_head // w.n_kv_head
    # the last block (few rows see it), one that ends on the tile before it, and one in the second half
    picks = [(w.batch - 1, w.n_kv_head - 1, S - 128), (0, 0, S - 384), (w.batch // 2, 1, (S // 2 // 128 + 3) * 128)]
    scale = 1.0 / np.sqrt(w.head_dim)
    for b, hkv, j0 in picks:
        want_k, want_v, want_q = _block_grads_f64(qn, kn, vn, dn, b, hkv, j0, j0 + 128, w.causal, scale)
        for got, want, what in ((d_k[b, hkv, j0:j0 + 128], want_k, "d_k"), (d_v[b, hkv, j0:j0 + 128], want_v, "d_v"),
                                (d_q[b, hkv * g_, j0:j0 + 128], want_q, "d_q")):
            gg = got.float().cpu().numpy()
            assert np.isfinite(gg).all(), (name, what, b, hkv, j0)
            err = np.abs(gg - want).max() / max(np.abs(want).max(), 1e-6)
            assert err <= GRAD_REL_TO_MAX, f"{name} {what} block (b={b}, kv head {hkv}, keys {j0}..): {err:.3e}"


def test_zero_extents_follow_autograd():
    # autograd of ATen's operator on the same shapes: no queries -> dK, dV are zeros; no keys -> dQ is zeros
    from tyr_b200 import nn as tnn
    dev = _dev()
    q = torch.empty(2, 4, 0, 64, dtype=torch.bfloat16, device=dev)
    k = torch.randn(2, 2, 33, 64, device=dev).bfloat16()
    o, lse = tnn.attentionFwd(q, k, k, is_causal=False)
    dq, dk, dv = tnn.attentionBwd(q, k, k, o, lse, torch.empty_like(q), is_causal=False)
    assert dq.numel() == 0 and not dk.any() and not dv.any() and dk.shape == k.shape
    q = torch.randn(2, 4, 5, 128, device=dev).bfloat16()
    k = torch.empty(2, 2, 0, 128, dtype=torch.bfloat16, device=dev)
    o, lse = tnn.attentionFwd(q, k, k, is_causal=False)
    dq, dk, dv = tnn.attentionBwd(q, k, k, o, lse, torch.randn_like(q), is_causal=False)
    assert not dq.any() and dq.shape == q.shape and dk.numel() == 0 and dv.numel() == 0
    qf = q.float().cpu().requires_grad_(True)
    kf = k.float().cpu().requires_grad_(True)
    ref = torch.nn.functional.scaled_dot_product_attention(qf, kf, kf, enable_gqa=True)
    ref.backward(torch.ones_like(ref))
    assert not qf.grad.any()
