"""The give-up path of the in-kernel barrier waits, exercised without faulting anything:
a one-warp kernel waits on a barrier nobody arrives at, with a limit of about a millisecond;
the wait returns false, the kernel records why and exits, and the library reports it."""
import time

import pytest
import torch

from tyr_b200 import _lib
from tyr_b200 import nn as tnn

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_a_stalled_wait_runs_out_and_is_reported():
    L = _lib.load()
    torch.cuda.set_device(0)
    assert tnn.device_status(0, True) >= 0
    stream = torch.cuda.current_stream().cuda_stream
    t0 = time.perf_counter()
    assert L.tyr_b200_attn_test_stalled_wait(2_000_000, stream) == 0      # about 1 ms of SM clocks
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 5.0                                  # it returned by itself
    assert tnn.device_status(0, False) & 1                                 # TYR_ATTN_STATUS_WAIT_TIMEOUT
    assert L.tyr_b200_attn_device_check(0) == -9                           # -TYR_ATTN_ERR_DEVICE_WAIT
    assert L.tyr_b200_attn_strerror(-9).startswith(b"tyr_b200_attn:")
    assert tnn.device_status(0, False) == 0                                # cleared by the check
    with pytest.raises(_lib.AttnError):
        assert L.tyr_b200_attn_test_stalled_wait(1_000_000, stream) == 0
        tnn.device_check(0)
    # the context is intact: a normal attention call afterwards is correct
    g = torch.Generator(device="cpu").manual_seed(0)
    q = torch.randn(1, 2, 200, 128, generator=g).bfloat16().to(DEV)
    o, lse = tnn.attentionFwd(q, q, q, is_causal=True)
    oc, lc = tnn.attentionFwd(q, q, q, is_causal=True, check_mode=True)
    assert (o.float() - oc.float()).abs().max().item() <= 2e-2
    assert tnn.device_status(0, True) == 0


def test_wait_limit_is_a_launch_parameter():
    """Shortening the limit for the attention kernels themselves must not disturb a healthy
    run (no legitimate wait comes near 50 ms), and the default comes back with 0."""
    L = _lib.load()
    L.tyr_b200_attn_test_set_wait_limit(100_000_000)
    try:
        g = torch.Generator(device="cpu").manual_seed(1)
        q = torch.randn(2, 4, 700, 128, generator=g).bfloat16().to(DEV)
        k = torch.randn(2, 2, 700, 128, generator=g).bfloat16().to(DEV)
        o, lse = tnn.attentionFwd(q, k, k, is_causal=True)
        d_o = torch.randn(2, 4, 700, 128, generator=g).bfloat16().to(DEV)
        tnn.attentionBwd(q, k, k, o, lse, d_o, is_causal=True)
        assert tnn.device_status(0, True) == 0
    finally:
        L.tyr_b200_attn_test_set_wait_limit(0)
