"""Parity of the sm_100a prefill kernels with the CPU oracle, through the C ABI."""
import ctypes

import numpy as np
import pytest
import torch

from conftest import CHECK_REL, LSE_REL, O_MAX_ABS
from oracle import c_oracle
from tyr_b200 import _lib, nn as tnn
from tyr_b200 import workloads as W

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def oracle(q, k, v, causal):
    """fp32 CPU result on the bf16-rounded values (Examples/GPU/RunFlashAttn.lean:30-36)."""
    return c_oracle.sdpa(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy(), causal)


def assert_parity(o, lse, ro, rlse, tag=""):
    o = o.float().cpu().numpy()
    assert not np.isnan(o).any(), tag
    assert np.abs(o - ro).max() <= O_MAX_ABS, (tag, float(np.abs(o - ro).max()))
    if lse is not None:
        lse = lse.cpu().numpy()
        err = np.abs(lse - rlse) / np.maximum(np.abs(rlse), 1.0)
        assert err.max() <= LSE_REL, (tag, float(err.max()))


def randn(*shape, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(*shape, generator=g).bfloat16()


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    assert tnn.device_status(0, True) == 0, "a bounded in-kernel wait gave up"


def test_golden_vectors(golden):
    for name, g in golden.items():
        causal, win = bool(g["meta"][6]), int(g["meta"][7])
        q, k, v = (torch.tensor(g[x]).bfloat16().to(DEV) for x in ("q", "k", "v"))
        o, lse = tnn.attentionFwd(q, k, v, is_causal=causal, window_size=win)
        assert_parity(o, None if win else lse, g["o"], g["lse"], name)
        # check mode on the same (bf16-exact) fp32 inputs
        qf, kf, vf = (torch.tensor(g[x]).to(DEV) for x in ("q", "k", "v"))
        o32, lse32 = tnn.attentionFwd(qf, kf, vf, is_causal=causal, check_mode=True, window_size=win)
        scale = np.abs(g["o"]).max()
        assert np.abs(o32.cpu().numpy() - g["o"]).max() / scale <= CHECK_REL, name
        if not win:
            assert (np.abs(lse32.cpu().numpy() - g["lse"]) / np.maximum(np.abs(g["lse"]), 1.0)).max() <= CHECK_REL, name


@pytest.mark.parametrize("S", [200, 257, 700, 1300])
@pytest.mark.parametrize("window", [1, 7, 64, 128, 129, 300, 5000])
@pytest.mark.parametrize("D", [64, 128])
def test_sliding_window(S, window, D):
    # lean_torch_sdpa_gqa_window (cc/src/tyr.cpp:3953-4018): j <= i and i - j < window
    q, k, v = randn(1, 4, S, D, seed=S + window), randn(1, 2, S, D, seed=S + 1), randn(1, 2, S, D, seed=S + 2)
    o, lse = tnn.attentionFwd(q.to(DEV), k.to(DEV), v.to(DEV), is_causal=True, window_size=window)
    ro, rlse = c_oracle.sdpa(q.float().numpy(), k.float().numpy(), v.float().numpy(), True, window=window)
    assert_parity(o, lse, ro, rlse, (S, window, D))
    o2 = tnn.scaledDotProductAttentionGQAWindow(q.to(DEV), k.to(DEV), v.to(DEV), 0.0, False, True, window)
    assert torch.equal(o2, o)       # the typed call ignores is_causal, like the reference


@pytest.mark.parametrize("S", [1, 63, 64, 65, 127, 128, 129, 255, 256, 257, 383, 512, 700])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("causal", [False, True])
def test_ragged_sequence_lengths(S, D, causal):
    q, k, v = randn(2, 4, S, D, seed=S), randn(2, 2, S, D, seed=S + 1), randn(2, 2, S, D, seed=S + 2)
    o, lse = tnn.attentionFwd(q.to(DEV), k.to(DEV), v.to(DEV), is_causal=causal)
    ro, rlse = oracle(q, k, v, causal)
    assert_parity(o, lse, ro, rlse, (S, D, causal))


@pytest.mark.parametrize("S", [150, 400, 1000])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("causal", [False, True])
def test_padding_key_mask(S, D, causal):
    # lean_torch_sdpa_gqa_mask (cc/src/tyr.cpp:4024-4095): 0 in the [batch, seq] mask hides that key
    B = 3
    q, k, v = randn(B, 4, S, D, seed=S), randn(B, 2, S, D, seed=S + 1), randn(B, 2, S, D, seed=S + 2)
    m = torch.ones(B, S, dtype=torch.uint8)
    m[0, S // 2:] = 0                 # right padding, whole KV tiles masked out for long S
    m[1, 5:S // 3] = 0                # a hole
    m[2, 1::2] = 0                    # every other key
    o, lse = tnn.attentionFwd(q.to(DEV), k.to(DEV), v.to(DEV), is_causal=causal, key_mask=m.to(DEV))
    ro, rlse = c_oracle.sdpa(q.float().numpy(), k.float().numpy(), v.float().numpy(), causal, key_mask=m.numpy())
    assert_parity(o, lse, ro, rlse, (S, D, causal))
    oc, lc = tnn.attentionFwd(q.to(DEV), k.to(DEV), v.to(DEV), is_causal=causal, key_mask=m.to(DEV), check_mode=True)
    assert_parity(oc, lc, ro, rlse, ("check", S, D, causal))
    o2 = tnn.scaledDotProductAttentionGQAMask(q.to(DEV), k.to(DEV), v.to(DEV), m.float().to(DEV), 0.0, causal, True)
    assert torch.equal(o2, o)


def test_padding_key_mask_golden_and_unseen_rows():
    import os
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "aten_keymask.npz"))
    f = lambda a: torch.tensor((a.astype(np.uint32) << 16).view(np.float32)).bfloat16().to(DEV)
    q, k, v, m = f(g["q"]), f(g["k"]), f(g["v"]), torch.tensor(g["mask"]).to(DEV)
    for causal, key in ((True, "o_causal"), (False, "o_full")):
        o, _ = tnn.attentionFwd(q, k, v, is_causal=causal, key_mask=m)
        assert_parity(o, None, g[key], None, key)
    # a query that sees no key at all gets NaN, like ATen's softmax over all -inf
    m0 = torch.ones(2, q.shape[2], dtype=torch.uint8)
    m0[:, 0] = 0
    o, _ = tnn.attentionFwd(q, k, v, is_causal=True, key_mask=m0.to(DEV))
    assert torch.isnan(o[:, :, 0].float()).all() and not torch.isnan(o[:, :, 1:].float()).any()


@pytest.mark.parametrize("Sq,Skv", [(1, 300), (5, 9), (100, 700), (300, 40), (129, 128)])
@pytest.mark.parametrize("causal", [False, True])
def test_query_and_key_lengths_differ(Sq, Skv, causal):
    # lean_torch_sdpa_gqa_qkv; causal is top-left aligned as in ATen (key j masked when j > i)
    q, k, v = randn(1, 4, Sq, 128, seed=1), randn(1, 1, Skv, 128, seed=2), randn(1, 1, Skv, 128, seed=3)
    o = tnn.scaledDotProductAttentionGQAQKV(q.to(DEV), k.to(DEV), v.to(DEV), 0.0, causal, True)
    ro, _ = oracle(q, k, v, causal)
    assert_parity(o, None, ro, None, (Sq, Skv, causal))


@pytest.mark.parametrize("Hq,Hkv", [(3, 1), (6, 2), (5, 5), (8, 1), (2, 2)])
@pytest.mark.parametrize("causal", [False, True])
def test_gqa_group_sizes(Hq, Hkv, causal):
    # even groups pair two heads of a KV head in one work item, odd groups pair row blocks
    S, D = 330, 128
    q, k, v = randn(2, Hq, S, D, seed=Hq), randn(2, Hkv, S, D, seed=Hq + 1), randn(2, Hkv, S, D, seed=Hq + 2)
    o, lse = tnn.attentionFwd(q.to(DEV), k.to(DEV), v.to(DEV), is_causal=causal)
    ro, rlse = oracle(q, k, v, causal)
    assert_parity(o, lse, ro, rlse, (Hq, Hkv, causal))


def test_random_shapes_against_the_fp32_kernel():
    """Seeded sweep over shapes, masks and strides: tensor-core kernel vs the fp32-FMA kernel."""
    rng = np.random.default_rng(2024)
    for case in range(40):
        D = int(rng.choice([64, 128]))
        Hkv = int(rng.integers(1, 4))
        g = int(rng.choice([1, 2, 3, 4]))
        B = int(rng.integers(1, 4))
        Sq = int(rng.integers(1, 900))
        same = bool(rng.integers(0, 2))
        Skv = Sq if same else int(rng.integers(1, 900))
        causal = bool(rng.integers(0, 2))
        window = int(rng.integers(1, 400)) if (same and rng.integers(0, 3) == 0) else 0
        use_mask = same and not window and rng.integers(0, 4) == 0
        q, k, v = randn(B, Hkv * g, Sq, D, seed=case), randn(B, Hkv, Skv, D, seed=case + 100), randn(B, Hkv, Skv, D, seed=case + 200)
        km = None
        if use_mask:
            km = torch.tensor(rng.integers(0, 2, (B, Skv)), dtype=torch.uint8)
            km[:, 0] = 1                      # every causal row keeps at least its first key
            km = km.to(DEV)
        kw = dict(is_causal=causal, window_size=window, key_mask=km)
        o, lse = tnn.attentionFwd(q.to(DEV), k.to(DEV), v.to(DEV), **kw)
        oc, lc = tnn.attentionFwd(q.to(DEV), k.to(DEV), v.to(DEV), check_mode=True, **kw)
        tag = (case, B, Hkv, g, Sq, Skv, D, causal, window, use_mask)
        assert not torch.isnan(o.float()).any(), tag
        assert (o.float() - oc.float()).abs().max().item() <= O_MAX_ABS, tag
        assert ((lse - lc).abs() / lc.abs().clamp(min=1.0)).max().item() <= LSE_REL, tag


def test_two_streams_do_not_interfere():
    q, k, v = randn(2, 4, 600, 128, seed=81).to(DEV), randn(2, 2, 600, 128, seed=82).to(DEV), randn(2, 2, 600, 128, seed=83).to(DEV)
    ref, ref_lse = tnn.attentionFwd(q, k, v, is_causal=True)
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    outs = []
    for st in (s1, s2, s1, s2):
        with torch.cuda.stream(st):
            outs.append(tnn.attentionFwd(q, k, v, is_causal=True))
    torch.cuda.synchronize()
    for o, l in outs:
        assert torch.equal(o, ref) and torch.equal(l, ref_lse)


def test_typed_calls_mirror_the_lean_externs():
    q, k, v = randn(2, 4, 200, 64, seed=7), randn(2, 4, 200, 64, seed=8), randn(2, 4, 200, 64, seed=9)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    o = tnn.scaled_dot_product_attention(qd, kd, vd)          # is_causal defaults to true
    assert_parity(o, None, oracle(q, k, v, True)[0], None)
    o = tnn.scaled_dot_product_attention(qd, kd, vd, 0.0, False)
    assert_parity(o, None, oracle(q, k, v, False)[0], None)
    kg, vg = k[:, :2].contiguous(), v[:, :2].contiguous()
    o = tnn.scaledDotProductAttentionGQA(qd, kg.to(DEV), vg.to(DEV), 0.0, True, True)
    assert_parity(o, None, oracle(q, kg, vg, True)[0], None)
    with pytest.raises(_lib.AttnError):                        # enable_gqa = false with fewer KV heads
        tnn.scaledDotProductAttentionGQA(qd, kg.to(DEV), vg.to(DEV), 0.0, True, False)
    with pytest.raises(_lib.AttnError):                        # dropout stays with LibTorch
        tnn.scaled_dot_product_attention(qd, kd, vd, 0.1, True)


def test_raw_c_abi_entry_points():
    L = _lib.load()
    q, k, v = randn(1, 4, 150, 128, seed=11), randn(1, 2, 150, 128, seed=12), randn(1, 2, 150, 128, seed=13)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    out = torch.empty_like(qd)
    st = torch.cuda.current_stream().cuda_stream
    rc = L.tyr_b200_sdpa_gqa(1, 4, 2, 150, 128, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(),
                             out.data_ptr(), 0.0, 1, 1, st)
    assert rc == 0
    assert_parity(out, None, oracle(q, k, v, True)[0], None)
    q1 = qd[:, :, -1:].contiguous()
    out1 = torch.empty_like(q1)
    rc = L.tyr_b200_sdpa_gqa_qkv(1, 4, 2, 1, 150, 128, q1.data_ptr(), kd.data_ptr(), vd.data_ptr(),
                                 out1.data_ptr(), 0.0, 0, 1, st)
    assert rc == 0
    # cached decode == last row of the causal prefill (Tests/TestQwen3Model.lean:36-55)
    assert (out1.float() - out[:, :, -1:].float()).abs().max().item() <= 1e-2
    k4, v4 = kd.repeat_interleave(2, 1), vd.repeat_interleave(2, 1)
    out4 = torch.empty_like(qd)
    assert L.tyr_b200_sdpa_4d(1, 4, 150, 128, qd.data_ptr(), k4.data_ptr(), v4.data_ptr(),
                              out4.data_ptr(), 0.0, 1, st) == 0
    assert torch.equal(out4, out)      # GQA index map == repeat_interleave, bit for bit


def test_strided_views_and_caller_allocated_outputs():
    # K/V as the slice of a larger cache (Tyr/Model/Qwen/Attention.lean:195-196)
    cap, L_ = 512, 300
    kc, vc = randn(2, 2, cap, 128, seed=21).to(DEV), randn(2, 2, cap, 128, seed=22).to(DEV)
    q = randn(2, 4, L_, 128, seed=23).to(DEV)
    k, v = kc[:, :, :L_], vc[:, :, :L_]
    assert not k.is_contiguous()
    out = torch.zeros(2, 4, L_, 128, dtype=torch.bfloat16, device=DEV)
    lse = torch.zeros(2, 4, L_, dtype=torch.float32, device=DEV)
    o2, lse2 = tnn.attentionFwd(q, k, v, is_causal=True, out=out, lse=lse)
    assert o2.data_ptr() == out.data_ptr()
    ro, rlse = oracle(q.cpu(), k.cpu(), v.cpu(), True)
    assert_parity(out, lse, ro, rlse)
    # [B,S,H,D] storage viewed as [B,H,S,D]
    qb = randn(2, 200, 4, 64, seed=24).to(DEV)
    kb, vb = randn(2, 200, 2, 64, seed=25).to(DEV), randn(2, 200, 2, 64, seed=26).to(DEV)
    ob = torch.empty(2, 200, 4, 64, dtype=torch.bfloat16, device=DEV)
    tnn.attentionFwd(qb.transpose(1, 2), kb.transpose(1, 2), vb.transpose(1, 2), is_causal=True,
                     out=ob.transpose(1, 2), return_lse=False)
    ro, _ = oracle(qb.transpose(1, 2).cpu(), kb.transpose(1, 2).cpu(), vb.transpose(1, 2).cpu(), True)
    assert_parity(ob.transpose(1, 2), None, ro, None)


@pytest.mark.parametrize("B,H,Hkv,S,D,causal", [(2, 6, 3, 777, 64, True), (1, 8, 2, 2048, 128, False),
                                                (3, 4, 4, 300, 128, True), (2, 15, 5, 1024, 64, False)])
def test_layout_does_not_change_a_bit(B, H, Hkv, S, D, causal):
    # [B,S,H,D] storage viewed as [B,H,S,D] against contiguous copies of the same values: the
    # kernels see the same tiles either way, so O and LSE must agree bit for bit
    q = randn(B, S, H, D, seed=61).to(DEV).transpose(1, 2)
    k, v = randn(B, S, Hkv, D, seed=62).to(DEV).transpose(1, 2), randn(B, S, Hkv, D, seed=63).to(DEV).transpose(1, 2)
    o1, l1 = tnn.attentionFwd(q, k, v, is_causal=causal)
    ob = torch.empty(B, S, H, D, dtype=torch.bfloat16, device=DEV)
    o2, l2 = tnn.attentionFwd(q.contiguous(), k.contiguous(), v.contiguous(), is_causal=causal, out=ob.transpose(1, 2))
    assert torch.equal(o1, o2) and torch.equal(l1, l2)
    oc, lc = tnn.attentionFwd(q, k, v, is_causal=causal, check_mode=True)
    oc2, lc2 = tnn.attentionFwd(q.contiguous(), k.contiguous(), v.contiguous(), is_causal=causal, check_mode=True)
    assert torch.equal(oc, oc2) and torch.equal(lc, lc2)


def test_rows_outside_the_tensor_are_not_written():
    S = 130
    q, k, v = randn(1, 2, S, 128, seed=31), randn(1, 2, S, 128, seed=32), randn(1, 2, S, 128, seed=33)
    big = torch.full((1, 2, S + 64, 128), 7.0, dtype=torch.bfloat16, device=DEV)
    tnn.attentionFwd(q.to(DEV), k.to(DEV), v.to(DEV), is_causal=False, out=big[:, :, :S], return_lse=False)
    assert (big[:, :, S:] == 7.0).all()


def test_large_logits_and_scale_argument():
    q, k, v = randn(1, 2, 256, 128, seed=41) * 6, randn(1, 2, 256, 128, seed=42) * 6, randn(1, 2, 256, 128, seed=43)
    o, lse = tnn.attentionFwd(q.to(DEV), k.to(DEV), v.to(DEV), is_causal=True)
    ro, rlse = oracle(q, k, v, True)
    assert_parity(o, lse, ro, rlse)
    o, lse = tnn.attentionFwd(q.to(DEV), k.to(DEV), v.to(DEV), is_causal=False, scale=0.01)
    ro, rlse = c_oracle.sdpa(q.float().numpy(), k.float().numpy(), v.float().numpy(), False, scale=0.01)
    assert_parity(o, lse, ro, rlse)


def test_check_mode_fp32_inputs_within_1e5():
    g = torch.Generator(device="cpu").manual_seed(51)
    q, k, v = (torch.randn(2, 4, 300, 96, generator=g) for _ in range(3))
    k, v = k[:, :2].contiguous(), v[:, :2].contiguous()
    o, lse = tnn.attentionFwd(q.to(DEV), k.to(DEV), v.to(DEV), is_causal=True, check_mode=True)
    ro, rlse = c_oracle.sdpa(q.numpy(), k.numpy(), v.numpy(), True)
    assert np.abs(o.cpu().numpy() - ro).max() / np.abs(ro).max() <= CHECK_REL
    assert (np.abs(lse.cpu().numpy() - rlse) / np.maximum(np.abs(rlse), 1.0)).max() <= CHECK_REL


@pytest.mark.parametrize("name,batch,heads,seq", [
    ("gpt_char", 4, (6, 6), None),               # configs[0] shape, fewer batches
    ("qwen3_0p6b_prefill", 1, (4, 2), 2048),     # configs[1] head geometry
    ("flux_mmdit", 1, (2, 2), 1152),             # configs[4], non-causal
])
def test_workload_shapes_against_oracle(name, batch, heads, seq):
    w = W.WORKLOADS[name]
    q, k, v = W.make_prefill(w, batch=batch, heads=heads, seq=seq)
    o, lse = tnn.attentionFwd(q.to(DEV), k.to(DEV), v.to(DEV), is_causal=w.causal)
    ro, rlse = oracle(q, k, v, w.causal)
    assert_parity(o, lse, ro, rlse, name)


def _sampled_rows_vs_oracle(q, k, v, o, lse, causal, n=48, seed=0):
    """Exact oracle answer for a sample of (b, h, row): the row only needs its own keys."""
    B, Hq, S, D = q.shape
    g = Hq // k.shape[1]
    rng = np.random.default_rng(seed)
    for _ in range(n):
        b, h, i = int(rng.integers(B)), int(rng.integers(Hq)), int(rng.integers(S))
        if _ % 8 == 0:
            i = min([0, S - 1, 127, 128, 255, 256, S // 2][(_ // 8) % 7], S - 1)
        n_keys = i + 1 if causal else k.shape[2]
        qr = q[b, h, i].float().cpu().numpy().reshape(1, 1, 1, D)
        kr = k[b, h // g, :n_keys].float().cpu().numpy().reshape(1, 1, n_keys, D)
        vr = v[b, h // g, :n_keys].float().cpu().numpy().reshape(1, 1, n_keys, D)
        ro, rl = c_oracle.sdpa(qr, kr, vr, False)
        assert np.abs(o[b, h, i].float().cpu().numpy() - ro[0, 0, 0]).max() <= O_MAX_ABS, (b, h, i)
        assert abs(lse[b, h, i].item() - rl[0, 0, 0]) / max(abs(rl[0, 0, 0]), 1.0) <= LSE_REL, (b, h, i)


@pytest.mark.parametrize("name", ["qwen3_0p6b_prefill", "qwen3_8b_prefill", "flux_mmdit", "gpt_char"])
def test_full_size_workloads_by_sampled_rows_and_properties(name):
    w = W.WORKLOADS[name]
    q, k, v = (t.to(DEV) for t in W.make_prefill(w))
    o, lse = tnn.attentionFwd(q, k, v, is_causal=w.causal)
    assert not torch.isnan(o.float()).any()
    _sampled_rows_vs_oracle(q, k, v, o, lse, w.causal)
    # property 1: the output is a convex combination of V rows
    vmax = v.float().abs().amax(dim=(2,), keepdim=True).repeat_interleave(w.n_head // w.n_kv_head, 1)
    assert (o.float().abs() <= vmax * 1.01 + 1e-3).all()
    # property 2: linear in V (same softmax weights): attn(2V) == 2 attn(V) up to bf16 rounding
    o2, lse2 = tnn.attentionFwd(q, k, v * 2, is_causal=w.causal)
    assert torch.equal(lse2, lse)
    assert (o2.float() - 2 * o.float()).abs().max().item() <= 2e-2
    # property 3: the tensor-core kernel agrees with the fp32-FMA kernel on one (batch, KV head)
    b, hk, g = w.batch - 1, w.n_kv_head - 1, w.n_head // w.n_kv_head
    qs = q[b:b + 1, hk * g:(hk + 1) * g]
    oc, lc = tnn.attentionFwd(qs, k[b:b + 1, hk:hk + 1], v[b:b + 1, hk:hk + 1], is_causal=w.causal,
                              check_mode=True)
    assert (oc.float() - o[b:b + 1, hk * g:(hk + 1) * g].float()).abs().max().item() <= O_MAX_ABS
    assert ((lc - lse[b:b + 1, hk * g:(hk + 1) * g]).abs() / lc.abs().clamp(min=1)).max().item() <= LSE_REL


def test_tabled_schedule_gives_the_static_schedule_bits():
    # A causal launch whose K/V exceed the L2 budget (items in several chunks) deals its items to the
    # CTAs by a host-built table; the same (batch, KV head) groups computed alone run the static
    # schedule.  An item's arithmetic does not depend on who runs it or when: identical bits.
    w = W.WORKLOADS["qwen3_8b_prefill"]
    q, k, v = (t.to(DEV) for t in W.make_prefill(w))
    o, lse = tnn.attentionFwd(q, k, v, is_causal=True)
    o_again, lse_again = tnn.attentionFwd(q, k, v, is_causal=True)      # the table is cached now
    assert torch.equal(o, o_again) and torch.equal(lse, lse_again)
    g = w.n_head // w.n_kv_head
    for b, hk in ((0, 0), (w.batch - 1, w.n_kv_head - 1), (1, 3)):
        os_, ls_ = tnn.attentionFwd(q[b:b + 1, hk * g:(hk + 1) * g], k[b:b + 1, hk:hk + 1], v[b:b + 1, hk:hk + 1],
                                    is_causal=True)
        assert torch.equal(os_, o[b:b + 1, hk * g:(hk + 1) * g]) and torch.equal(ls_, lse[b:b + 1, hk * g:(hk + 1) * g])


def test_graph_capture_of_a_call_that_would_build_a_table():
    # a new launch geometry met for the first time on a capturing stream: no table is built (that
    # would allocate and copy synchronously), the static schedule is captured, and the replay gives
    # the bits of the eager call that follows (which does build the table)
    q, k, v = (randn(3, 8, 8192, 128, seed=s).to(DEV) for s in (11, 12, 13))
    o, lse = torch.empty_like(q), torch.empty(q.shape[:3], device=DEV)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            tnn.attentionFwd(q, k, v, is_causal=True, out=o, lse=lse)
    torch.cuda.current_stream().wait_stream(side)
    o.zero_()
    graph.replay()
    torch.cuda.synchronize()
    o_eager, lse_eager = tnn.attentionFwd(q, k, v, is_causal=True)
    assert torch.equal(o, o_eager) and torch.equal(lse, lse_eager)
    _sampled_rows_vs_oracle(q, k, v, o, lse, True, n=16, seed=3)


def test_merge_entry_point_against_oracle_and_full_attention():
    q, k, v = randn(1, 2, 64, 128, seed=61), randn(1, 2, 600, 128, seed=62), randn(1, 2, 600, 128, seed=63)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    oa, la = tnn.attentionFwd(qd, kd[:, :, :256], vd[:, :, :256], is_causal=False)
    ob, lb = tnn.attentionFwd(qd, kd[:, :, 256:], vd[:, :, 256:], is_causal=False)
    om, lm = tnn.mergePartials(oa.float().reshape(-1, 128), la.reshape(-1), ob.float().reshape(-1, 128),
                               lb.reshape(-1))
    ro, rl = c_oracle.merge2(oa.float().cpu().numpy().reshape(-1, 128), la.cpu().numpy().reshape(-1),
                             ob.float().cpu().numpy().reshape(-1, 128), lb.cpu().numpy().reshape(-1))
    assert np.abs(om.cpu().numpy() - ro).max() <= 1e-5
    assert np.abs(lm.cpu().numpy() - rl).max() <= 1e-5
    fo, fl = oracle(q, k, v, False)
    assert np.abs(om.cpu().numpy().reshape(fo.shape) - fo).max() <= O_MAX_ABS
    assert np.abs(lm.cpu().numpy().reshape(fl.shape) - fl).max() <= 1e-3 * np.abs(fl).max()


def test_host_buffer_call():
    q, k, v = randn(2, 4, 300, 128, seed=71), randn(2, 2, 300, 128, seed=72), randn(2, 2, 300, 128, seed=73)
    qp, kp, vp = q.pin_memory(), k.pin_memory(), v.pin_memory()
    lse = torch.empty(2, 4, 300, dtype=torch.float32).pin_memory()
    o, lse = tnn.sdpa_host(qp, kp, vp, is_causal=True, lse=lse)
    assert not o.is_cuda
    ro, rlse = oracle(q, k, v, True)
    assert_parity(o, lse, ro, rlse)


def test_launches_are_counted():
    n0 = tnn.launch_count()
    q = randn(1, 1, 64, 64).to(DEV)
    tnn.attentionFwd(q, q, q)
    assert tnn.launch_count() == n0 + 1


def test_zero_extents_follow_aten():
    # ATen's operator on the same shapes: an empty output for an empty batch / query, zeros without keys
    for shape_q, shape_k in (((0, 4, 16, 64), (0, 2, 16, 64)), ((2, 4, 0, 64), (2, 2, 16, 64))):
        q, k = torch.empty(shape_q, dtype=torch.bfloat16, device=DEV), randn(*shape_k).to(DEV) if shape_k[0] else \
            torch.empty(shape_k, dtype=torch.bfloat16, device=DEV)
        o, lse = tnn.attentionFwd(q, k, k, is_causal=False)
        assert tuple(o.shape) == shape_q and tuple(lse.shape) == shape_q[:3]
    q = randn(2, 4, 5, 128).to(DEV)
    k = torch.empty(2, 2, 0, 128, dtype=torch.bfloat16, device=DEV)
    base = torch.full((2, 5, 4, 128), float("nan"), dtype=torch.bfloat16, device=DEV)
    out = base.transpose(1, 2)                      # a strided output view
    o, lse = tnn.attentionFwd(q, k, k, is_causal=False, out=out)
    ref = torch.nn.functional.scaled_dot_product_attention(q.float().cpu(), k.float().cpu(), k.float().cpu(), enable_gqa=True)
    assert torch.equal(o.float().cpu(), ref) and not ref.any()
    assert torch.isneginf(lse).all()


def test_calls_from_several_threads_on_their_own_streams():
    # Lean may call from any task thread (no global state in the reference's entry points): three threads,
    # each on its own stream; two of them meet a geometry that builds a schedule table on first use
    # (causal, K/V beyond the L2 budget), at the same time
    import threading
    shapes = [((5, 8, 8192, 128), (5, 8, 8192, 128), True), ((3, 12, 6144, 128), (3, 12, 6144, 128), True),
              ((2, 4, 700, 64), (2, 4, 700, 64), False)]
    inputs = [(randn(*sq, seed=70 + i).to(DEV), randn(*sk, seed=80 + i).to(DEV), randn(*sk, seed=90 + i).to(DEV), c)
              for i, (sq, sk, c) in enumerate(shapes)]
    got, errs = [None] * len(shapes), []

    def work(i):
        try:
            q, k, v, c = inputs[i]
            st = torch.cuda.Stream(device=DEV)
            with torch.cuda.stream(st):
                for _ in range(20):
                    o, lse = tnn.attentionFwd(q, k, v, is_causal=c)
                st.synchronize()
            got[i] = (o, lse)
        except Exception as e:  # surfaced below: an exception in a thread would otherwise pass silently
            errs.append(e)

    threads = [threading.Thread(target=work, args=(i,)) for i in range(len(shapes))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errs, errs
    torch.cuda.synchronize()
    for (o, lse), (q, k, v, c) in zip(got, inputs):
        wo, wl = tnn.attentionFwd(q, k, v, is_causal=c)
        assert torch.equal(o, wo) and torch.equal(lse, wl)
    # and against the oracle on one (batch, head) of the first
    q, k, v, _ = inputs[0]
    ro, rl = oracle(q[4:5, 7:8, :1024].cpu(), k[4:5, 7:8, :1024].cpu(), v[4:5, 7:8, :1024].cpu(), True)
    assert_parity(got[0][0][4:5, 7:8, :1024], got[0][1][4:5, 7:8, :1024], ro, rl)
