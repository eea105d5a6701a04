"""Calls on a second GPU of the same process: per-device state (status word, kernel attributes, schedule
tables, the static decode scratch, staging buffers of the host-buffer call) must follow the tensors' device,
not the thread's current one.  Skipped on a one-GPU box."""
import pytest
import torch

from oracle import c_oracle
from tyr_b200 import nn as tnn

pytestmark = pytest.mark.gpu


def randn(*shape, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(*shape, generator=g).bfloat16()


@pytest.fixture(autouse=True)
def _two_devices():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs in one process")
    torch.cuda.set_device(0)
    yield
    for d in (0, 1):
        assert tnn.device_status(d, True) == 0


def test_forward_backward_on_the_other_device_match_the_first():
    q, k, v = randn(2, 8, 640, 128, seed=1), randn(2, 4, 640, 128, seed=2), randn(2, 4, 640, 128, seed=3)
    d_o = randn(2, 8, 640, 128, seed=4)
    res = []
    for dev in ("cuda:0", "cuda:1"):
        qd, kd, vd, dd = (t.to(dev) for t in (q, k, v, d_o))
        o, lse = tnn.attentionFwd(qd, kd, vd, is_causal=True)        # current device stays 0 throughout
        grads = tnn.attentionBwd(qd, kd, vd, o, lse, dd, is_causal=True)
        res.append([t.cpu() for t in (o, lse, *grads)])
    assert torch.cuda.current_device() == 0
    for a, b in zip(*res):
        assert torch.equal(a, b)
    ro, rl = c_oracle.sdpa(q.float().numpy(), k.float().numpy(), v.float().numpy(), True)
    assert abs(res[1][0].float().numpy() - ro).max() <= 2e-2


def test_tabled_schedule_and_key_split_on_the_other_device():
    dev = "cuda:1"
    q, k, v = (randn(5, 8, 8192, 128, seed=s).to(dev) for s in (5, 6, 7))   # causal, K/V beyond the L2 budget
    o, lse = tnn.attentionFwd(q, k, v, is_causal=True)
    o1, l1 = tnn.attentionFwd(q[4:5, 7:8], k[4:5, 7:8], v[4:5, 7:8], is_causal=True)   # static schedule
    assert torch.equal(o[4:5, 7:8], o1) and torch.equal(lse[4:5, 7:8], l1)
    q, k, v = (randn(1, 12, 3584, 128, seed=s).to(dev) for s in (8, 9, 10))  # 168 items: a thin last round
    os_, ls_ = tnn.attentionFwd(q, k, v, is_causal=False)                     # allocates the workspace itself
    on, ln = tnn.attentionFwd(q, k, v, is_causal=False, workspace=False)
    assert (os_.float() - on.float()).abs().max().item() <= 2e-2
    assert ((ls_ - ln).abs() / ln.abs().clamp(min=1)).max().item() <= 1e-3


def test_decode_and_host_call_on_the_other_device():
    dev = "cuda:1"
    lens = [5, 700, 4100]
    ks = [randn(2, L, 128, seed=20 + i).to(dev) for i, L in enumerate(lens)]
    vs = [randn(2, L, 128, seed=30 + i).to(dev) for i, L in enumerate(lens)]
    q = randn(3, 8, 128, seed=40).to(dev)
    plan = tnn.DecodePlan(ks, vs, 8)
    o, lse = tnn.flashDecode(q, plan)
    o2, l2 = tnn.flashDecodeStatic(q, plan)
    assert torch.equal(o, o2) and torch.equal(lse, l2)
    for b, L in enumerate(lens):
        ro, rl = c_oracle.sdpa(q[b:b + 1, :, None].float().cpu().numpy(), ks[b][None].float().cpu().numpy(),
                               vs[b][None].float().cpu().numpy(), False)
        assert abs(o[b].float().cpu().numpy() - ro[0, :, 0]).max() <= 2e-2
    qh, kh, vh = randn(2, 4, 300, 64, seed=50), randn(2, 2, 300, 64, seed=51), randn(2, 2, 300, 64, seed=52)
    oh, _ = tnn.sdpa_host(qh, kh, vh, is_causal=True, device=1)
    od, _ = tnn.attentionFwd(qh.to(dev), kh.to(dev), vh.to(dev), is_causal=True)
    assert torch.equal(oh, od.cpu())
    assert torch.cuda.current_device() == 0
