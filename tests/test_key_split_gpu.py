"""The key-split of a half-empty last round (TyrAttnPrefillArgs.workspace) against the oracle and the unsplit kernel."""
import numpy as np
import pytest
import torch

from conftest import LSE_REL, O_MAX_ABS
from oracle import c_oracle
from tyr_b200 import nn as tnn

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def randn(*shape, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(*shape, generator=g).bfloat16()


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    assert tnn.device_status(0, True) == 0, "a bounded in-kernel wait gave up"


def _close_to_unsplit(q, k, v, o, lse):
    o0, lse0 = tnn.attentionFwd(q, k, v, is_causal=False, workspace=False)
    assert (o.float() - o0.float()).abs().max().item() <= O_MAX_ABS / 2
    if lse is not None:
        assert ((lse - lse0).abs() / lse0.abs().clamp(min=1.0)).max().item() <= LSE_REL


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("Sq,Skv", [(2048, 2048), (300, 2000), (128, 1024), (1, 1500), (200, 1100)])
def test_single_round_is_split_and_matches_the_oracle(D, Sq, Skv):
    q, k, v = randn(1, 4, Sq, D, seed=Sq + D), randn(1, 2, Skv, D, seed=Skv + 1), randn(1, 2, Skv, D, seed=Skv + 2)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    assert tnn.prefill_workspace_bytes(qd, kd, vd, is_causal=False) > 0
    assert tnn.prefill_workspace_bytes(qd, kd, vd, is_causal=True) == 0     # causal launches are never split
    n0 = tnn.launch_count()
    o, lse = tnn.attentionFwd(qd, kd, vd, is_causal=False)
    assert tnn.launch_count() - n0 == 2                                      # the kernel and the merge
    ro, rlse = c_oracle.sdpa(q.float().numpy(), k.float().numpy(), v.float().numpy(), False)
    assert np.abs(o.float().cpu().numpy() - ro).max() <= O_MAX_ABS
    assert (np.abs(lse.cpu().numpy() - rlse) / np.maximum(np.abs(rlse), 1.0)).max() <= LSE_REL
    _close_to_unsplit(qd, kd, vd, o, lse)


@pytest.mark.parametrize("B,H,Skv,parts", [(1, 8, 2304, 4), (2, 20, 2304, 3), (4, 16, 2304, 2), (1, 8, 4200, 8), (1, 24, 4096, 6)])
def test_more_than_two_parts(B, H, Skv, parts):
    # few items against many SMs (148): 8 items of 18 KV tiles -> 4 parts each, 40 -> 3, 64 -> 2,
    # 8 items of 33 tiles -> 8, 24 items -> 6
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    items = B * H
    if min(sms // items, 8, ((Skv + 127) // 128) // 4) != parts:
        pytest.skip("this device's SM count gives another number of parts")
    q, k, v = (randn(B, H, 256, 128, seed=3 + H).to(DEV), randn(B, H, Skv, 128, seed=4 + H).to(DEV),
               randn(B, H, Skv, 128, seed=5 + H).to(DEV))
    need = tnn.prefill_workspace_bytes(q, k, v, is_causal=False)
    assert need == items * parts * 2 * 128 * (128 * 2 + 4)
    o, lse = tnn.attentionFwd(q, k, v, is_causal=False)
    _close_to_unsplit(q, k, v, o, lse)
    ro, rlse = c_oracle.sdpa(q[:1, :2].float().cpu().numpy(), k[:1, :2].float().cpu().numpy(),
                             v[:1, :2].float().cpu().numpy(), False)
    assert np.abs(o[:1, :2].float().cpu().numpy() - ro).max() <= O_MAX_ABS
    assert (np.abs(lse[:1, :2].cpu().numpy() - rlse) / np.maximum(np.abs(rlse), 1.0)).max() <= LSE_REL


def test_last_of_two_rounds_is_split():
    # 12 heads x 14 row blocks of 256 = 168 items on 148 SMs: 20 items in the second round
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    q, k, v = (randn(1, 12, 3584, 128, seed=s).to(DEV) for s in (1, 2, 3))
    need = tnn.prefill_workspace_bytes(q, k, v, is_causal=False)
    rem = 168 % sms
    if rem == 0 or 2 * rem > sms:
        pytest.skip("this device's SM count leaves no half-empty round for 168 items")
    parts = min(sms // rem, 8, 28 // 4)   # as many parts as fit the SMs, at least four KV tiles each
    assert need == rem * parts * 2 * 128 * (128 * 2 + 4)
    o, lse = tnn.attentionFwd(q, k, v, is_causal=False)
    _close_to_unsplit(q, k, v, o, lse)
    # exact rows of the split items (the lowest row blocks come last in the item order) and of others
    rows = [0, 1, 127, 128, 255, 256, 300, 511, 2000, 3583]
    qs = q[0, :, rows].float().cpu().numpy()[None].transpose(0, 1, 2, 3)
    ro, rlse = c_oracle.sdpa(qs, k.float().cpu().numpy(), v.float().cpu().numpy(), False)
    assert np.abs(o[0, :, rows].float().cpu().numpy() - ro[0]).max() <= O_MAX_ABS
    assert (np.abs(lse[0, :, rows].cpu().numpy() - rlse[0]) / np.maximum(np.abs(rlse[0]), 1.0)).max() <= LSE_REL


def test_strided_output_no_lse_and_caller_workspace():
    q, k, v = (randn(2, 2, 1024, 128, seed=s).to(DEV) for s in (4, 5, 6))
    need = tnn.prefill_workspace_bytes(q, k, v, is_causal=False)
    assert need > 0
    ws = torch.empty(need + 256, dtype=torch.uint8, device=DEV)
    buf = torch.full((2, 1024, 2, 128), 7.0, dtype=torch.bfloat16, device=DEV)   # [B,S,H,D] storage
    out = buf.permute(0, 2, 1, 3)
    o, lse = tnn.attentionFwd(q, k, v, is_causal=False, out=out, return_lse=False, workspace=ws)
    assert lse is None and o.data_ptr() == buf.data_ptr()
    _close_to_unsplit(q, k, v, o, None)
    # a workspace that is too small is ignored: the call runs unsplit
    n0 = tnn.launch_count()
    o2, _ = tnn.attentionFwd(q, k, v, is_causal=False, workspace=ws[:256])
    assert tnn.launch_count() - n0 == 1
    _close_to_unsplit(q, k, v, o2, None)
    with pytest.raises(ValueError):
        tnn.attentionFwd(q, k, v, is_causal=False, workspace=ws[1:])
