"""The allocation-free decode entry point against the regular one (collected last).

Some callers of this library cannot allocate device memory while they decode
(their pool owns the device, or an allocation's synchronisation would stall the
token loop).  tyr_b200_attn_decode_static serves them from a fixed 16 MiB array
inside the library.  It must give what tyr_b200_attn_decode gives, call after
call, although the array keeps whatever the previous call left in it.
"""
import pytest
import torch

import numpy as np

from conftest import LSE_REL, O_MAX_ABS
from oracle import c_oracle
from tyr_b200 import _lib, nn as tnn

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def randn(*shape, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(*shape, generator=g).bfloat16().to(DEV)


def make_case(lens, seed, n_head=8, n_kv_head=2, d=128):
    ks = [randn(n_kv_head, L, d, seed=seed + i) for i, L in enumerate(lens)]
    vs = [randn(n_kv_head, L, d, seed=seed + 100 + i) for i, L in enumerate(lens)]
    q = randn(len(lens), n_head, d, seed=seed + 999)
    return q, tnn.DecodePlan(ks, vs, n_head)


def assert_oracle(q, plan, o, lse):
    """The result of the allocation-free entry against the CPU oracle, sequence by sequence."""
    ks, vs = plan._keep
    for b in range(q.shape[0]):
        Hq, D = q.shape[1], q.shape[2]
        ro, rl = c_oracle.sdpa(q[b].float().cpu().numpy().reshape(1, Hq, 1, D), ks[b].float().cpu().numpy()[None],
                               vs[b].float().cpu().numpy()[None], False)
        assert np.abs(o[b].float().cpu().numpy() - ro[0, :, 0]).max() <= O_MAX_ABS
        err = np.abs(lse[b].cpu().numpy() - rl[0, :, 0]) / np.maximum(np.abs(rl[0, :, 0]), 1.0)
        assert err.max() <= LSE_REL


def assert_same(o, lse, ro, rlse):
    assert not torch.isnan(o.float()).any()
    assert (o.float() - ro.float()).abs().max().item() <= O_MAX_ABS
    assert ((lse - rlse).abs() / rlse.abs().clamp(min=1.0)).max().item() <= LSE_REL


def test_static_scratch_decode_matches_workspace_decode_twice_in_a_row():
    # call 1: long sequences, many chunks -> the array is filled with partials
    q1, plan1 = make_case([4000, 9000, 700, 12000], seed=1)
    ref1 = tnn.flashDecode(q1, plan1)
    got1 = tnn.flashDecodeStatic(q1, plan1)
    assert_same(*got1, *ref1)
    assert_oracle(q1, plan1, *got1)
    # call 2, straight after, other data and other chunk counts: stale partials of
    # call 1 are still in the array and must not leak into the result
    q2, plan2 = make_case([2500, 300, 6000], seed=2, n_head=16, n_kv_head=4)
    got2 = tnn.flashDecodeStatic(q2, plan2)
    ref2 = tnn.flashDecode(q2, plan2)
    assert_same(*got2, *ref2)
    assert_oracle(q2, plan2, *got2)
    # and the first case again gives the first answer again
    got1b = tnn.flashDecodeStatic(q1, plan1)
    assert torch.equal(got1b[0], got1[0]) and torch.equal(got1b[1], got1[1])
    assert tnn.device_status(0, True) == 0


def test_static_scratch_decode_refuses_sizes_beyond_its_array():
    L = _lib.load()
    # 64 sequences x 32 heads x 64 chunks x 129 floats = 67 MB of partials > 16 MiB
    assert L.tyr_b200_attn_decode_workspace_bytes(64, 32, 128, 32768, 64) > _lib.DECODE_STATIC_SCRATCH_BYTES
    a = _lib.DecodeArgs()
    a.batch, a.n_head, a.n_kv_head, a.max_kv_seq, a.head_dim = 64, 32, 8, 32768, 128
    import ctypes
    rc = L.tyr_b200_attn_decode_static(ctypes.byref(a), None)
    assert rc == -10
    assert b"maximum" in L.tyr_b200_attn_strerror(rc)
