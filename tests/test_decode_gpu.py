"""Parity of split-KV flash-decoding with the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from conftest import LSE_REL, O_MAX_ABS
from oracle import c_oracle
from tyr_b200 import nn as tnn
from tyr_b200 import workloads as W

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def randn(*shape, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(*shape, generator=g).bfloat16()


def check_seq(q_b, k_b, v_b, o_b, lse_b, tag=""):
    """q_b [Hq,D]; k_b, v_b [Hkv,L,D]: the per-sequence call of forwardStep, on the oracle."""
    Hq, D = q_b.shape
    ro, rl = c_oracle.sdpa(q_b.float().cpu().numpy().reshape(1, Hq, 1, D),
                           k_b.float().cpu().numpy()[None], v_b.float().cpu().numpy()[None], False)
    o = o_b.float().cpu().numpy()
    assert not np.isnan(o).any(), tag
    assert np.abs(o - ro[0, :, 0]).max() <= O_MAX_ABS, (tag, float(np.abs(o - ro[0, :, 0]).max()))
    err = np.abs(lse_b.cpu().numpy() - rl[0, :, 0]) / np.maximum(np.abs(rl[0, :, 0]), 1.0)
    assert err.max() <= LSE_REL, (tag, float(err.max()))


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("Hq,Hkv", [(8, 2), (4, 4), (32, 8), (40, 2)])
def test_ragged_lengths(D, Hq, Hkv):
    lens = [1, 2, 15, 16, 17, 63, 64, 65, 255, 256, 257, 511, 513, 1000, 3000]
    ks = [randn(Hkv, L, D, seed=L).to(DEV) for L in lens]
    vs = [randn(Hkv, L, D, seed=L + 7).to(DEV) for L in lens]
    q = randn(len(lens), Hq, D, seed=99).to(DEV)
    plan = tnn.DecodePlan(ks, vs, Hq)
    o, lse = tnn.flashDecode(q, plan)
    for b, L in enumerate(lens):
        check_seq(q[b], ks[b], vs[b], o[b], lse[b], (D, Hq, Hkv, L))


@pytest.mark.parametrize("max_splits", [1, 3, 64])
def test_split_count_does_not_change_the_answer(max_splits):
    lens = [700, 5000, 9000]
    ks = [randn(2, L, 128, seed=L).to(DEV) for L in lens]
    vs = [randn(2, L, 128, seed=L + 1).to(DEV) for L in lens]
    q = randn(3, 8, 128, seed=5).to(DEV)
    o, lse = tnn.flashDecode(q, tnn.DecodePlan(ks, vs, 8, max_splits=max_splits))
    for b in range(3):
        check_seq(q[b], ks[b], vs[b], o[b], lse[b], (max_splits, b))


@pytest.mark.parametrize("lens", [[9000], [4100, 300, 7000], [2500] * 6])
def test_length_hint_only_steers_the_chunks(lens):
    # total_kv_len (the sum the host knows) lets a small launch cut its chunks for one wave of CTAs;
    # without it, or with a sum that cannot be right, the answer stays within the same bars
    Hq, Hkv, D = 8, 2, 128
    ks = [randn(Hkv, L, D, seed=L).to(DEV) for L in lens]
    vs = [randn(Hkv, L, D, seed=L + 3).to(DEV) for L in lens]
    q = randn(len(lens), Hq, D, seed=5).to(DEV)
    plan = tnn.DecodePlan(ks, vs, Hq)
    assert plan.total_kv_len == sum(lens)
    for hint in (sum(lens), 0, 1, 10 ** 12):
        plan.total_kv_len = hint
        o, lse = tnn.flashDecode(q, plan)
        for b in range(len(lens)):
            check_seq(q[b], ks[b], vs[b], o[b], lse[b], f"hint {hint} seq {b}")
    assert tnn.device_status(0, True) == 0


def test_dense_cache_layout_and_4d_query():
    # Tyr's KVCache: [batch, n_kv_head, maxLen, head_dim] with a shared `seq` counter
    B, Hq, Hkv, cap, D, kv_len = 3, 8, 2, 1024, 128, 777
    kc, vc = randn(B, Hkv, cap, D, seed=1).to(DEV), randn(B, Hkv, cap, D, seed=2).to(DEV)
    kc[:, :, kv_len:] = float("nan")      # slots past the counter must never be read
    vc[:, :, kv_len:] = float("nan")
    q = randn(B, Hq, 1, D, seed=3).to(DEV)
    o, lse = tnn.flashDecodeDense(q, kc, vc, kv_len=kv_len)
    for b in range(B):
        check_seq(q[b, :, 0], kc[b, :, :kv_len], vc[b, :, :kv_len], o[b], lse[b], b)
    lens = torch.tensor([5, 300, 1024], dtype=torch.int32, device=DEV)
    kc, vc = randn(B, Hkv, cap, D, seed=4).to(DEV), randn(B, Hkv, cap, D, seed=5).to(DEV)
    o, lse = tnn.flashDecodeDense(q, kc, vc, kv_lens=lens)
    for b, L in enumerate(lens.tolist()):
        check_seq(q[b, :, 0], kc[b, :, :L], vc[b, :, :L], o[b], lse[b], b)


def test_decode_equals_last_row_of_causal_prefill():
    # cached vs uncached parity, the model-level pin of Tests/TestQwen3Model.lean:36-55
    S, Hq, Hkv, D = 900, 8, 2, 128
    q, k, v = randn(1, Hq, S, D, seed=11).to(DEV), randn(1, Hkv, S, D, seed=12).to(DEV), randn(1, Hkv, S, D, seed=13).to(DEV)
    o_full, lse_full = tnn.attentionFwd(q, k, v, is_causal=True)
    o, lse = tnn.flashDecode(q[:, :, -1].contiguous(), tnn.DecodePlan([k[0]], [v[0]], Hq))
    assert (o.float() - o_full[:, :, -1].float()).abs().max().item() <= 1e-2
    assert (lse - lse_full[:, :, -1]).abs().max().item() <= 1e-3 * lse_full.abs().max().item()


def test_workspace_is_required_for_split_runs():
    from tyr_b200 import _lib
    ks, vs = [randn(2, 4000, 128).to(DEV)], [randn(2, 4000, 128, seed=1).to(DEV)]
    plan = tnn.DecodePlan(ks, vs, 8)
    plan.workspace_bytes = 16
    with pytest.raises(_lib.AttnError):
        tnn.flashDecode(randn(1, 8, 128).to(DEV), plan)


def test_full_size_decode_workload():
    """configs[3]: 64 ragged sequences in [512, 32768]; every sequence against the oracle."""
    w = W.WORKLOADS["qwen3_8b_decode"]
    q, ks, vs, lens = W.make_decode(w, device=DEV)
    assert len(lens) == 64 and min(lens) >= 512 and max(lens) <= 32768
    q = q.to(DEV)
    plan = tnn.DecodePlan(ks, vs, w.n_head)
    o, lse = tnn.flashDecode(q, plan)
    assert tnn.device_status(0, True) == 0
    for b in range(0, 64, 3):
        check_seq(q[b], ks[b], vs[b], o[b], lse[b], (b, lens[b]))
    # idempotence: same inputs, same bits (split order is fixed)
    o2, lse2 = tnn.flashDecode(q, plan)
    assert torch.equal(o, o2) and torch.equal(lse, lse2)


def test_lengths_outside_the_limits_are_clamped_and_reported():
    """kv_lens above max_kv_seq would index past the grid and the workspace; the kernels clamp
    them, a length of zero gives a defined row, and the status word says so."""
    B, Hq, Hkv, cap, D = 3, 8, 2, 600, 128
    kc, vc = randn(B, Hkv, cap, D, seed=11).to(DEV), randn(B, Hkv, cap, D, seed=12).to(DEV)
    q = randn(B, Hq, D, seed=13).to(DEV)
    tnn.device_status(0, True)
    lens = torch.tensor([300, 100000, 0], dtype=torch.int32, device=DEV)
    o, lse = tnn.flashDecodeDense(q, kc, vc, kv_lens=lens, kv_len=512)
    assert tnn.device_status(0, True) & 4
    check_seq(q[0], kc[0, :, :300], vc[0, :, :300], o[0], lse[0], "in range")
    check_seq(q[1], kc[1, :, :512], vc[1, :, :512], o[1], lse[1], "clamped to max_kv_seq")
    assert (o[2] == 0).all() and torch.isinf(lse[2]).all() and (lse[2] < 0).all()
    # in-range lengths leave the status word alone
    lens = torch.tensor([300, 512, 1], dtype=torch.int32, device=DEV)
    tnn.flashDecodeDense(q, kc, vc, kv_lens=lens, kv_len=512)
    assert tnn.device_status(0, True) == 0


def test_decode_plan_rejects_misaligned_blocks():
    base = torch.zeros(2 * 70 * 128 + 64, dtype=torch.bfloat16, device=DEV)
    good = base[:2 * 70 * 128].view(2, 70, 128)
    tnn.DecodePlan([good], [good], 8)
    shifted = base[4:4 + 2 * 70 * 128].view(2, 70, 128)           # 8 bytes off a 16-byte boundary
    with pytest.raises(ValueError):
        tnn.DecodePlan([shifted], [shifted], 8)
    odd_stride = torch.as_strided(base, (2, 70, 128), (70 * 128 + 4, 128, 1))   # head stride not a multiple of 8
    with pytest.raises(ValueError):
        tnn.DecodePlan([odd_stride], [odd_stride], 8)
