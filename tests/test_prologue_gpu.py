"""Fused RMSNorm + rotary + layout + KV-append kernel against the oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from oracle import c_oracle
from tyr_b200 import nn as tnn

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
# one bf16 rounding of an fp32 result: half an ulp relative, plus the fp32 arithmetic itself
BF16_REL = 2.0 ** -8


def rope_tables(max_pos, d, base=10000.0):
    inv = 1.0 / (base ** (torch.arange(0, d // 2).float() / (d // 2)))
    ang = torch.arange(max_pos).float()[:, None] * inv[None]
    return ang.cos().contiguous(), ang.sin().contiguous()


def close(got, ref):
    got = got.float().cpu().numpy()
    assert not np.isnan(got).any()
    assert (np.abs(got - ref) <= BF16_REL * np.abs(ref) + 1e-6).all(), float(np.abs(got - ref).max())


@pytest.mark.parametrize("D", [64, 128, 256])
@pytest.mark.parametrize("use_norm,use_rope", [(True, True), (True, False), (False, True), (False, False)])
def test_against_oracle(D, use_norm, use_rope):
    g = torch.Generator(device="cpu").manual_seed(D)
    B, S, H, cap = 3, 7, 4, 32
    x = torch.randn(B, S, H, D, generator=g).bfloat16()
    w = (torch.rand(D, generator=g) + 0.5) if use_norm else None
    cos, sin = rope_tables(cap, D) if use_rope else (None, None)
    pos = torch.tensor([0, 5, 25], dtype=torch.int32)
    cache = torch.randn(B, H, cap, D, generator=g).bfloat16()
    ref = cache.float().numpy().copy()
    c_oracle.qk_prologue(x.float().numpy(), ref, None if w is None else w.numpy(),
                         None if cos is None else cos.numpy(), None if sin is None else sin.numpy(),
                         positions=pos.numpy())
    out = cache.to(DEV)
    tnn.qkPrologue(x.to(DEV), out, None if w is None else w.to(DEV), None if cos is None else cos.to(DEV),
                   None if sin is None else sin.to(DEV), positions=pos.to(DEV))
    close(out, ref)
    # untouched rows of the cache are bit-identical
    mask = torch.ones(B, cap, dtype=torch.bool)
    for b, p0 in enumerate(pos.tolist()):
        mask[b, p0:p0 + S] = False
    assert torch.equal(out.cpu().transpose(1, 2)[mask], cache.transpose(1, 2)[mask])


def test_golden_reference_chain():
    import os
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "aten_prologue.npz"))
    start = int(g["start"])
    out = torch.tensor(g["cache"]).bfloat16().to(DEV)
    tnn.qkPrologue(torch.tensor(g["x"]).bfloat16().to(DEV), out, torch.tensor(g["w"]).to(DEV),
                   torch.tensor(g["cos"]).to(DEV), torch.tensor(g["sin"]).to(DEV), position0=start)
    S = g["x"].shape[1]
    close(out[:, :, start:start + S], g["new_cache"][:, :, start:start + S])


def test_decode_step_through_prologue_and_flash_decode():
    """One token of QwenAttention.forwardStep after the projections
    (Tyr/Model/Qwen/Attention.lean:151-200): head norm, rotary, cache append, attention."""
    g = torch.Generator(device="cpu").manual_seed(3)
    B, Hq, Hkv, D, cap, seq = 2, 8, 2, 128, 300, 257
    kc = torch.randn(B, Hkv, cap, D, generator=g).bfloat16()
    vc = torch.randn(B, Hkv, cap, D, generator=g).bfloat16()
    kc[:, :, seq:] = float("nan")
    vc[:, :, seq:] = float("nan")
    q = torch.randn(B, 1, Hq, D, generator=g).bfloat16()
    k = torch.randn(B, 1, Hkv, D, generator=g).bfloat16()
    v = torch.randn(B, 1, Hkv, D, generator=g).bfloat16()
    qn, kn = torch.rand(D, generator=g) + 0.5, torch.rand(D, generator=g) + 0.5
    cos, sin = rope_tables(cap, D)
    # oracle: the same steps on fp32
    kref, vref = kc.float().numpy().copy(), vc.float().numpy().copy()
    c_oracle.qk_prologue(k.float().numpy(), kref, kn.numpy(), cos.numpy(), sin.numpy(), position0=seq)
    c_oracle.qk_prologue(v.float().numpy(), vref, position0=seq)
    qref = np.zeros((B, Hq, 1, D), np.float32)
    c_oracle.qk_prologue(q.float().numpy(), qref, qn.numpy(), cos.numpy()[seq:], sin.numpy()[seq:])
    bf = lambda a: torch.tensor(a).bfloat16().float().numpy()          # tensors are bf16 between ops
    oref, _ = c_oracle.sdpa(bf(qref), bf(kref[:, :, :seq + 1]), bf(vref[:, :, :seq + 1]), False)
    # device: three prologue launches and one decode launch, cache updated in place
    kd, vd = kc.to(DEV), vc.to(DEV)
    tnn.qkPrologue(k.to(DEV), kd, kn.to(DEV), cos.to(DEV), sin.to(DEV), position0=seq)
    tnn.qkPrologue(v.to(DEV), vd, position0=seq)
    qd = torch.empty(B, Hq, 1, D, dtype=torch.bfloat16, device=DEV)
    tnn.qkPrologue(q.to(DEV), qd, qn.to(DEV), cos[seq:].contiguous().to(DEV), sin[seq:].contiguous().to(DEV))
    o, _ = tnn.flashDecodeDense(qd, kd, vd, kv_len=seq + 1)
    assert np.abs(o.float().cpu().numpy() - oref[:, :, 0]).max() <= 2e-2


def test_rejects_bad_arguments():
    from tyr_b200 import _lib
    x = torch.zeros(1, 1, 1, 96, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(1, 1, 4, 96, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(_lib.AttnError):
        tnn.qkPrologue(x, out)


def test_cache_limit_rows_are_skipped_and_reported():
    """A row that would land past the cache (the reference guards its append with
    `cache.seq < cache.maxLen`, Tyr/Model/Qwen/Attention.lean:189) is never written: the kernel
    skips it and raises the out-of-range bit; a guard region after the cache stays intact."""
    from tyr_b200 import _lib
    g = torch.Generator(device="cpu").manual_seed(17)
    B, S, H, D, cap = 2, 4, 2, 128, 8
    x = torch.randn(B, S, H, D, generator=g).bfloat16()
    # one allocation: the cache of B*H*cap rows followed by a guard region of sentinels
    store = torch.full((B * H * cap + 64, D), 7.0, dtype=torch.bfloat16, device=DEV)
    cache = store[:B * H * cap].view(B, H, cap, D)
    cos, sin = rope_tables(cap, D)
    tnn.device_status(0, True)
    # sequence 0 fits exactly (rows 4..7); sequence 1 starts at 6: rows 8, 9 do not exist
    pos = torch.tensor([4, 6], dtype=torch.int32)
    ref = cache.float().cpu().numpy().copy()
    tnn.qkPrologue(x.to(DEV), cache, None, cos.to(DEV), sin.to(DEV), positions=pos.to(DEV))
    assert tnn.device_status(0, False) & 4
    with pytest.raises(_lib.AttnError):
        tnn.device_check(0)
    assert tnn.device_status(0, True) == 0          # device_check cleared it
    assert (store[B * H * cap:] == 7.0).all()       # guard untouched
    c_oracle.qk_prologue(x[:1].float().numpy(), ref[:1], None, cos.numpy(), sin.numpy(), position0=4)
    c_oracle.qk_prologue(x[1:, :2].float().numpy(), ref[1:], None, cos.numpy(), sin.numpy(), position0=6)
    close(cache, ref)
    # with the position known on the host the call is refused before any launch
    with pytest.raises(ValueError):
        tnn.qkPrologue(x.to(DEV), cache, position0=6)
    with pytest.raises(ValueError):
        tnn.qkPrologue(x.to(DEV), cache, None, cos[:7].contiguous().to(DEV), sin[:7].contiguous().to(DEV), position0=4)


@pytest.mark.parametrize("D", [64, 128, 256])
@pytest.mark.parametrize("shared_table", [False, True])
def test_flux_rotary_form_against_oracle(D, shared_table):
    g = torch.Generator(device="cpu").manual_seed(D + 1)
    B, S, H, cap = 2, 9, 5, 16
    x = torch.randn(B, S, H, D, generator=g).bfloat16()
    w = torch.rand(D, generator=g) + 0.5
    ang = torch.rand(1 if shared_table else B, cap, D // 2, generator=g) * 6.0
    pe = torch.stack([torch.stack([ang.cos(), -ang.sin()], -1), torch.stack([ang.sin(), ang.cos()], -1)], -2).contiguous()
    ref = np.zeros((B, H, cap, D), np.float32)
    c_oracle.qk_prologue_pe(x.float().numpy(), ref, pe.numpy(), weight=w.numpy(), position0=3)
    out = torch.zeros(B, H, cap, D, dtype=torch.bfloat16, device=DEV)
    tnn.qkPrologue(x.to(DEV), out, w.to(DEV), position0=3, pe=pe.to(DEV))
    close(out, ref)


def test_flux_rotary_golden_chain():
    """QKNorm + flux.applyRope + transpose as torch runs them (tests/golden/make_golden.py fluxrope)."""
    import os
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "aten_flux_rope.npz"))
    B, S, H, D = g["x"].shape
    out = torch.zeros(B, H, S, D, dtype=torch.bfloat16, device=DEV)
    pe = torch.tensor(g["pe"]).reshape(B, S, D // 2, 2, 2).contiguous()
    tnn.qkPrologue(torch.tensor(g["x"]).bfloat16().to(DEV), out, torch.tensor(g["w"]).to(DEV), pe=pe.to(DEV))
    close(out, g["y"])


def test_many_heads_and_ragged_token_count():
    # head counts that are not a multiple of the heads kept in flight, token counts that leave lane groups idle
    g = torch.Generator(device="cpu").manual_seed(23)
    for (B, S, H, D) in [(1, 1, 1, 128), (2, 3, 7, 64), (1, 5, 9, 256), (3, 33, 6, 128)]:
        x = torch.randn(B, S, H, D, generator=g).bfloat16()
        w = torch.rand(D, generator=g) + 0.5
        cos, sin = rope_tables(S + 2, D)
        ref = np.zeros((B, H, S + 2, D), np.float32)
        c_oracle.qk_prologue(x.float().numpy(), ref, w.numpy(), cos.numpy(), sin.numpy(), position0=2)
        out = torch.zeros(B, H, S + 2, D, dtype=torch.bfloat16, device=DEV)
        tnn.qkPrologue(x.to(DEV), out, w.to(DEV), cos.to(DEV), sin.to(DEV), position0=2)
        close(out, ref)


def test_query_of_a_decode_step_is_rotated_at_its_position_and_stored_at_row_zero():
    g = torch.Generator(device="cpu").manual_seed(29)
    B, H, D, max_pos = 3, 4, 128, 64
    x = torch.randn(B, 1, H, D, generator=g).bfloat16()
    w = torch.rand(D, generator=g) + 0.5
    cos, sin = rope_tables(max_pos, D)
    pos = torch.tensor([0, 17, 63], dtype=torch.int32)
    # oracle: write each sequence at its own position of a tall tensor, then read that row
    tall = np.zeros((B, H, max_pos, D), np.float32)
    c_oracle.qk_prologue(x.float().numpy(), tall, w.numpy(), cos.numpy(), sin.numpy(), positions=pos.numpy())
    ref = np.stack([tall[b, :, int(pos[b])] for b in range(B)])[:, :, None, :]
    out = torch.zeros(B, H, 1, D, dtype=torch.bfloat16, device=DEV)
    tnn.qkPrologue(x.to(DEV), out, w.to(DEV), cos.to(DEV), sin.to(DEV), positions=pos.to(DEV), out_at_row0=True)
    close(out, ref)
    assert tnn.device_status(0, True) == 0


def test_token_loop_captured_in_a_cuda_graph():
    """The decode step above as a serving loop would run it: the three prologue launches, the length
    update and the decode launch captured once into a CUDA graph and replayed per token, with the
    per-sequence lengths living on the device.  Every replay must give the bits of the same step run
    eagerly, and the last one is checked against the oracle."""
    g = torch.Generator(device="cpu").manual_seed(5)
    B, Hq, Hkv, D, cap, steps = 2, 8, 2, 128, 4400, 4
    start = [3, 4200]                                    # one sequence in a single chunk, one split over chunks
    kc = torch.randn(B, Hkv, cap, D, generator=g).bfloat16().to(DEV)
    vc = torch.randn(B, Hkv, cap, D, generator=g).bfloat16().to(DEV)
    toks = [[torch.randn(B, 1, h, D, generator=g).bfloat16().to(DEV) for h in (Hq, Hkv, Hkv)] for _ in range(steps)]
    qn, kn = (torch.rand(D, generator=g) + 0.5).to(DEV), (torch.rand(D, generator=g) + 0.5).to(DEV)
    cos, sin = (t.to(DEV) for t in rope_tables(cap, D))
    ws = torch.empty(tnn._lib.load().tyr_b200_attn_decode_workspace_bytes(B, Hq, D, cap, 64), dtype=torch.uint8, device=DEV)

    def step(q_in, k_in, v_in, kcache, vcache, lens, lens_next, qd):
        tnn.qkPrologue(k_in, kcache, kn, cos, sin, positions=lens)
        tnn.qkPrologue(v_in, vcache, positions=lens)
        tnn.qkPrologue(q_in, qd, qn, cos, sin, positions=lens, out_at_row0=True)
        torch.add(lens, 1, out=lens_next)
        o, lse = tnn.flashDecodeDense(qd, kcache, vcache, kv_lens=lens_next, kv_len=cap, workspace=ws)
        lens.copy_(lens_next)
        return o, lse

    # eager run on copies of the caches
    ke, ve = kc.clone(), vc.clone()
    lens_e = torch.tensor(start, dtype=torch.int32, device=DEV)
    nxt_e, qd_e = torch.empty_like(lens_e), torch.empty(B, Hq, 1, D, dtype=torch.bfloat16, device=DEV)
    eager = []
    for q_in, k_in, v_in in toks:
        o, lse = step(q_in, k_in, v_in, ke, ve, lens_e, nxt_e, qd_e)
        eager.append((o.clone(), lse.clone()))
    # captured run: static input buffers, one capture, one replay per token
    kg, vg = kc.clone(), vc.clone()
    lens_g = torch.tensor(start, dtype=torch.int32, device=DEV)
    nxt_g, qd_g = torch.empty_like(lens_g), torch.empty(B, Hq, 1, D, dtype=torch.bfloat16, device=DEV)
    q_s, k_s, v_s = (torch.empty_like(t) for t in toks[0])
    tnn.flashDecodeDense(qd_g.zero_(), kg, vg, kv_len=1, workspace=ws)      # loads the kernels outside the capture
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            o_g, lse_g = step(q_s, k_s, v_s, kg, vg, lens_g, nxt_g, qd_g)
    for (q_in, k_in, v_in), (oe, le) in zip(toks, eager):
        q_s.copy_(q_in); k_s.copy_(k_in); v_s.copy_(v_in)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(o_g, oe) and torch.equal(lse_g, le)
    assert torch.equal(kg, ke) and torch.equal(vg, ve) and lens_g.tolist() == [s + steps for s in start]
    assert tnn.device_status(0, True) == 0
    # the last token against the oracle, sequence by sequence
    for b, s0 in enumerate(start):
        L = s0 + steps
        ro, _ = c_oracle.sdpa(qd_g[b:b + 1].float().cpu().numpy(), kg[b:b + 1, :, :L].float().cpu().numpy(),
                              vg[b:b + 1, :, :L].float().cpu().numpy(), False)
        assert np.abs(o_g[b].float().cpu().numpy() - ro[0, :, 0]).max() <= 2e-2
