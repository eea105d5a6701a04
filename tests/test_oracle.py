"""The CPU oracle against the committed ATen outputs and closed-form cases (no GPU)."""
import numpy as np
import pytest
import torch

from oracle import aten_path, c_oracle


def rel(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def test_oracle_matches_golden_aten_outputs(golden):
    assert len(golden) >= 6
    for name, g in golden.items():
        causal, win = bool(g["meta"][6]), int(g["meta"][7])
        o, lse = c_oracle.sdpa(g["q"], g["k"], g["v"], causal, window=win)
        assert rel(o, g["o"]) < 1e-5, name
        if not win:      # ATen returns no LSE for the masked (windowed) call
            assert rel(lse, g["lse"]) < 1e-5, name


def test_golden_still_matches_this_torch(golden):
    # the fixtures were produced by the ATen operator; a torch upgrade that moved them would show here
    g = golden["qwen_gqa_causal"]
    o = aten_path.sdpa_gqa(torch.tensor(g["q"]), torch.tensor(g["k"]), torch.tensor(g["v"]), 0.0, True, True)
    assert rel(o.numpy(), g["o"]) < 1e-5


def test_online_form_equals_direct_form(golden):
    for name, g in golden.items():
        if int(g["meta"][7]):
            continue
        causal = bool(g["meta"][6])
        o, lse = c_oracle.sdpa(g["q"], g["k"], g["v"], causal)
        for block in (1, 7, 64):
            o2, lse2 = c_oracle.sdpa(g["q"], g["k"], g["v"], causal, online_block=block)
            assert rel(o2, o) < 2e-5, (name, block)
            assert rel(lse2, lse) < 2e-5, (name, block)


def test_single_key_softmax_is_identity():
    # closed form used by the reference's seq=1 attention test
    # (Tests/TestQwen35Model.lean:179-227): one key => weights == 1 => O == V, LSE == score
    rng = np.random.default_rng(1)
    q = rng.standard_normal((2, 4, 1, 32), dtype=np.float32)
    k = rng.standard_normal((2, 2, 1, 32), dtype=np.float32)
    v = rng.standard_normal((2, 2, 1, 32), dtype=np.float32)
    o, lse = c_oracle.sdpa(q, k, v, False)
    np.testing.assert_allclose(o, np.repeat(v, 2, axis=1), rtol=1e-6)
    s = (q * np.repeat(k, 2, axis=1)).sum(-1) / np.sqrt(32.0)
    np.testing.assert_allclose(lse, s, rtol=1e-5, atol=1e-6)


def test_equal_keys_give_mean_of_values():
    q = np.ones((1, 1, 3, 16), np.float32)
    k = np.ones((1, 1, 10, 16), np.float32)
    v = np.arange(160, dtype=np.float32).reshape(1, 1, 10, 16)
    o, lse = c_oracle.sdpa(q, k, v, False)
    np.testing.assert_allclose(o[0, 0, 0], v[0, 0].mean(0), rtol=1e-6)
    np.testing.assert_allclose(lse, 4.0 + np.log(10.0), rtol=1e-6)   # 16/sqrt(16) + log n
    o, lse = c_oracle.sdpa(q, k, v, True)                             # row i sees keys 0..i
    np.testing.assert_allclose(o[0, 0, 2], v[0, 0, :3].mean(0), rtol=1e-6)
    np.testing.assert_allclose(lse[0, 0], 4.0 + np.log([1.0, 2.0, 3.0]), rtol=1e-6)


def test_gqa_equals_repeat_interleave():
    rng = np.random.default_rng(2)
    q = rng.standard_normal((1, 6, 20, 32), dtype=np.float32)
    k = rng.standard_normal((1, 2, 20, 32), dtype=np.float32)
    v = rng.standard_normal((1, 2, 20, 32), dtype=np.float32)
    o, lse = c_oracle.sdpa(q, k, v, True)
    o2, lse2 = c_oracle.sdpa(q, np.repeat(k, 3, axis=1), np.repeat(v, 3, axis=1), True)
    np.testing.assert_array_equal(o, o2)
    np.testing.assert_array_equal(lse, lse2)


def test_merge_of_key_halves_equals_full_attention():
    rng = np.random.default_rng(3)
    q = rng.standard_normal((1, 2, 5, 64), dtype=np.float32)
    k = rng.standard_normal((1, 2, 50, 64), dtype=np.float32)
    v = rng.standard_normal((1, 2, 50, 64), dtype=np.float32)
    o, lse = c_oracle.sdpa(q, k, v, False)
    oa, la = c_oracle.sdpa(q, k[:, :, :20], v[:, :, :20], False)
    ob, lb = c_oracle.sdpa(q, k[:, :, 20:], v[:, :, 20:], False)
    om, lm = c_oracle.merge2(oa.reshape(-1, 64), la.reshape(-1), ob.reshape(-1, 64), lb.reshape(-1))
    assert rel(om.reshape(o.shape), o) < 1e-6
    assert rel(lm.reshape(lse.shape), lse) < 1e-6


def test_decode_step_equals_last_row_of_causal_prefill():
    # cached decode == uncached prefill, the parity the reference pins at model level
    # (Tests/TestQwen3Model.lean:36-55)
    rng = np.random.default_rng(4)
    q = rng.standard_normal((2, 4, 33, 64), dtype=np.float32)
    k = rng.standard_normal((2, 2, 33, 64), dtype=np.float32)
    v = rng.standard_normal((2, 2, 33, 64), dtype=np.float32)
    o, lse = c_oracle.sdpa(q, k, v, True)
    o1, lse1 = c_oracle.sdpa(q[:, :, -1:], k, v, False)
    assert rel(o1, o[:, :, -1:]) < 1e-6
    assert rel(lse1, lse[:, :, -1:]) < 1e-6


def test_bf16_round_matches_torch():
    rng = np.random.default_rng(5)
    x = np.concatenate([rng.standard_normal(4096).astype(np.float32) * 100,
                        np.array([0.0, -0.0, 1.0, 65504.0, 1e-40, np.inf, -np.inf], np.float32)])
    ref = torch.tensor(x).bfloat16().float().numpy()
    np.testing.assert_array_equal(c_oracle.bf16_round(x), ref)


def test_oracle_rejects_bad_shapes():
    q = np.zeros((1, 3, 2, 8), np.float32)
    k = np.zeros((1, 2, 2, 8), np.float32)
    with pytest.raises(ValueError):
        c_oracle.sdpa(q, k, k, False)


def test_prologue_oracle_matches_golden_reference_chain():
    import os
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "aten_prologue.npz"))
    cache = g["cache"].copy()
    start = int(g["start"])
    c_oracle.qk_prologue(g["x"], cache, g["w"], g["cos"], g["sin"], position0=start)
    assert rel(cache, g["new_cache"]) < 1e-6
    # rows outside [start, start + S) are the old cache, bit for bit
    S = g["x"].shape[1]
    keep = np.ones(cache.shape[2], bool)
    keep[start:start + S] = False
    np.testing.assert_array_equal(cache[:, :, keep], g["cache"][:, :, keep])


def test_prologue_oracle_parts():
    rng = np.random.default_rng(7)
    x = rng.standard_normal((1, 2, 2, 64), dtype=np.float32)
    out = np.zeros((1, 2, 4, 64), np.float32)
    c_oracle.qk_prologue(x, out, positions=[1])                      # plain transpose + append
    np.testing.assert_array_equal(out[0, :, 1:3], x[0].transpose(1, 0, 2))
    assert (out[0, :, 0] == 0).all() and (out[0, :, 3] == 0).all()
    w = np.ones(64, np.float32)
    out2 = np.zeros((1, 2, 2, 64), np.float32)
    c_oracle.qk_prologue(x, out2, weight=w)                          # unit RMS per head vector
    np.testing.assert_allclose((out2 ** 2).mean(-1), 1.0, rtol=1e-4)
    cos = np.zeros((2, 32), np.float32)
    sin = np.ones((2, 32), np.float32)                               # quarter turn: [x1,x2] -> [-x2,x1]
    out3 = np.zeros((1, 2, 2, 64), np.float32)
    c_oracle.qk_prologue(x, out3, cos=cos, sin=sin)
    xt = x[0].transpose(1, 0, 2)
    np.testing.assert_allclose(out3[0, :, :, :32], -xt[:, :, 32:], rtol=1e-6)
    np.testing.assert_allclose(out3[0, :, :, 32:], xt[:, :, :32], rtol=1e-6)


def test_window_closed_forms():
    rng = np.random.default_rng(11)
    q = rng.standard_normal((1, 2, 40, 32), dtype=np.float32)
    k = rng.standard_normal((1, 2, 40, 32), dtype=np.float32)
    v = rng.standard_normal((1, 2, 40, 32), dtype=np.float32)
    o, lse = c_oracle.sdpa(q, k, v, True, window=1)          # each query sees only its own key
    np.testing.assert_allclose(o, v, rtol=1e-6)
    np.testing.assert_allclose(lse, (q * k).sum(-1) / np.sqrt(32.0), rtol=1e-5, atol=1e-6)
    o_full, lse_full = c_oracle.sdpa(q, k, v, True)
    o_w, lse_w = c_oracle.sdpa(q, k, v, True, window=40)     # window >= seq is plain causal
    np.testing.assert_array_equal(o_w, o_full)
    np.testing.assert_array_equal(lse_w, lse_full)
    o5, _ = c_oracle.sdpa(q, k, v, True, window=5)           # row i == causal attention on keys i-4..i
    i = 20
    oi, _ = c_oracle.sdpa(q[:, :, i:i + 1], k[:, :, i - 4:i + 1], v[:, :, i - 4:i + 1], False)
    np.testing.assert_allclose(o5[:, :, i:i + 1], oi, rtol=1e-5, atol=1e-6)


def _load_keymask_golden():
    import os
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "aten_keymask.npz"))
    f = lambda a: (a.astype(np.uint32) << 16).view(np.float32)
    return f(g["q"]), f(g["k"]), f(g["v"]), g["mask"], g["o_causal"], g["o_full"]


def test_keymask_oracle_matches_golden_reference_mask():
    q, k, v, m, o_causal, o_full = _load_keymask_golden()
    o, _ = c_oracle.sdpa(q, k, v, True, key_mask=m)
    assert rel(o, o_causal) < 1e-5
    o, _ = c_oracle.sdpa(q, k, v, False, key_mask=m)
    assert rel(o, o_full) < 1e-5


def test_keymask_closed_forms():
    rng = np.random.default_rng(13)
    q = rng.standard_normal((1, 1, 6, 16), dtype=np.float32)
    k = rng.standard_normal((1, 1, 6, 16), dtype=np.float32)
    v = rng.standard_normal((1, 1, 6, 16), dtype=np.float32)
    m = np.array([[1, 1, 1, 0, 0, 0]], np.uint8)
    o, lse = c_oracle.sdpa(q, k, v, False, key_mask=m)           # == attention over the 3 valid keys
    o3, lse3 = c_oracle.sdpa(q, k[:, :, :3], v[:, :, :3], False)
    np.testing.assert_allclose(o, o3, rtol=1e-6)
    np.testing.assert_allclose(lse, lse3, rtol=1e-6)
    m0 = np.array([[0, 1, 1, 1, 1, 1]], np.uint8)                # causal row 0 sees only a padding key
    o, _ = c_oracle.sdpa(q, k, v, True, key_mask=m0)
    assert np.isnan(o[0, 0, 0]).all() and not np.isnan(o[0, 0, 1:]).any()


def test_backward_oracle_matches_golden_autograd(golden_backward):
    """The C restatement of the backward reproduces the stored torch-autograd gradients."""
    for name, c in golden_backward.items():
        B, Hq, Hkv, Sq, Skv, D, causal = (int(x) for x in c["meta"])
        d_q, d_k, d_v = c_oracle.sdpa_backward(c["q"], c["k"], c["v"], c["d_o"], bool(causal))
        for got, key in ((d_q, "d_q"), (d_k, "d_k"), (d_v, "d_v")):
            np.testing.assert_allclose(got, c[key], rtol=0, atol=2e-5, err_msg=f"{name}.{key}")


def test_backward_golden_still_matches_this_torch(golden_backward):
    c = golden_backward["gqa_causal"]
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    d_q, d_k, d_v = aten_path.sdpa_gqa_backward(t(c["q"]), t(c["k"]), t(c["v"]), t(c["d_o"]), True)
    for got, key in ((d_q, "d_q"), (d_k, "d_k"), (d_v, "d_v")):
        np.testing.assert_allclose(got.numpy(), c[key], rtol=0, atol=2e-5)


def test_backward_oracle_against_finite_differences():
    """d/dx of sum(O * dO) by central differences on a tiny case (fp64 would be exact to 1e-9;
    the fp32 interface limits this check to a few 1e-3)."""
    rng = np.random.default_rng(5)
    B, Hq, Hkv, Sq, Skv, D = 1, 2, 1, 5, 7, 4
    q, k, v, d_o = (rng.standard_normal(s).astype(np.float32) for s in
                    ((B, Hq, Sq, D), (B, Hkv, Skv, D), (B, Hkv, Skv, D), (B, Hq, Sq, D)))
    d_q, d_k, d_v = c_oracle.sdpa_backward(q, k, v, d_o, True)
    loss = lambda q_, k_, v_: float((c_oracle.sdpa(q_, k_, v_, True)[0].astype(np.float64) * d_o).sum())
    eps = 1e-2
    for arr, grad, which in ((q, d_q, 0), (k, d_k, 1), (v, d_v, 2)):
        for idx in [(0, 0, 1, 2), (0, arr.shape[1] - 1, 3, 0)]:
            plus, minus = arr.copy(), arr.copy()
            plus[idx] += eps
            minus[idx] -= eps
            args_p = [q, k, v]
            args_m = [q, k, v]
            args_p[which], args_m[which] = plus, minus
            fd = (loss(*args_p) - loss(*args_m)) / (2 * eps)
            assert abs(fd - grad[idx]) < 5e-3, (which, idx, fd, grad[idx])


def test_backward_of_a_single_key_is_closed_form():
    """One key: P = 1, so dV = sum of dO rows, dQ = 0, dK = 0."""
    rng = np.random.default_rng(6)
    q, d_o = rng.standard_normal((1, 2, 3, 8)).astype(np.float32), rng.standard_normal((1, 2, 3, 8)).astype(np.float32)
    k, v = rng.standard_normal((1, 1, 1, 8)).astype(np.float32), rng.standard_normal((1, 1, 1, 8)).astype(np.float32)
    d_q, d_k, d_v = c_oracle.sdpa_backward(q, k, v, d_o, False)
    np.testing.assert_allclose(d_q, 0, atol=1e-6)
    np.testing.assert_allclose(d_k, 0, atol=1e-6)
    np.testing.assert_allclose(d_v[0, 0, 0], d_o.sum(axis=(0, 1, 2)), rtol=1e-5, atol=1e-6)


def test_masked_backward_oracle_matches_autograd():
    """Sliding-window and padding-mask backward of the C oracle against torch autograd through the restated
    lean_torch_sdpa_gqa_window / lean_torch_sdpa_gqa_mask."""
    g = torch.Generator().manual_seed(31)
    B, Hq, Hkv, S, D = 2, 4, 2, 45, 16
    q, d_o = (torch.randn(B, Hq, S, D, generator=g) for _ in range(2))
    k, v = (torch.randn(B, Hkv, S, D, generator=g) for _ in range(2))
    want = aten_path.sdpa_gqa_backward(q, k, v, d_o, True, window=7)
    got = c_oracle.sdpa_backward(q.numpy(), k.numpy(), v.numpy(), d_o.numpy(), True, window=7)
    for a, b in zip(got, want):
        np.testing.assert_allclose(a, b.numpy(), rtol=0, atol=2e-5)
    m = torch.ones(B, S)
    m[0, 30:] = 0
    m[1, 5:12] = 0
    for causal in (True, False):
        want = aten_path.sdpa_gqa_backward(q, k, v, d_o, causal, padding_mask=m)
        got = c_oracle.sdpa_backward(q.numpy(), k.numpy(), v.numpy(), d_o.numpy(), causal, key_mask=m.numpy())
        for a, b in zip(got, want):
            np.testing.assert_allclose(a, b.numpy(), rtol=0, atol=2e-5)
        assert np.count_nonzero(got[1][0, :, 30:]) == 0 and np.count_nonzero(got[2][1, :, 5:12]) == 0


def test_flux_rotary_prologue_matches_the_torch_chain():
    """tyr_oracle_qk_prologue_pe against QKNorm + flux.applyRope + transpose as torch runs them
    (tests/golden/aten_flux_rope.npz, written by tests/golden/make_golden.py fluxrope)."""
    import os
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "aten_flux_rope.npz"))
    B, S, H, D = g["x"].shape
    out = np.zeros((B, H, S, D), np.float32)
    c_oracle.qk_prologue_pe(g["x"], out, g["pe"].reshape(B, S, D // 2, 2, 2), weight=g["w"])
    assert np.abs(out - g["y"]).max() <= 1e-5
    # a rotation by angle 0 is the identity (no weight: plain copy into the attention layout)
    ident = np.zeros((1, S, D // 2, 2, 2), np.float32)
    ident[..., 0, 0] = ident[..., 1, 1] = 1.0
    out2 = np.zeros((B, H, S, D), np.float32)
    c_oracle.qk_prologue_pe(g["x"], out2, ident)
    assert np.array_equal(out2, np.transpose(g["x"], (0, 2, 1, 3)))
