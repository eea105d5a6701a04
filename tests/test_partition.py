"""Sharding rules and the optional replicated-output gather (gloo, world_size 2, CPU)."""
import os
import socket
import subprocess
import sys
import textwrap

import pytest
import torch

from tyr_b200 import partition as P
from tyr_b200 import workloads as W

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("name,world,axis,b,h", [
    ("gpt_char", 8, "batch", 8, 6), ("gpt_char", 2, "heads", 64, 3),
    ("qwen3_0p6b_prefill", 8, "heads", 8, 1), ("qwen3_0p6b_prefill", 4, "heads", 8, 2),
    ("qwen3_8b_prefill", 8, "heads", 4, 1), ("qwen3_8b_prefill", 2, "heads", 4, 4),
    ("flux_mmdit", 8, "heads", 4, 3), ("flux_mmdit", 4, "heads", 4, 6),
])
def test_prefill_shards_follow_the_scope_table(name, world, axis, b, h):
    w = W.WORKLOADS[name]
    seen = set()
    for r in range(world):
        s = P.prefill_shard(w.batch, w.n_kv_head, world, r)
        assert s.axis == axis
        assert s.batch[1] - s.batch[0] == b and s.kv_heads[1] - s.kv_heads[0] == h
        for bi in range(*s.batch):
            for hi in range(*s.kv_heads):
                assert (bi, hi) not in seen
                seen.add((bi, hi))
    assert len(seen) == w.batch * w.n_kv_head          # every unit exactly once


def test_grid_split_when_neither_axis_divides():
    shards = [P.prefill_shard(4, 6, 8, r) for r in range(8)]
    assert {s.axis for s in shards} == {"batch*heads"}
    units = [(b, h) for s in shards for b in range(*s.batch) for h in range(*s.kv_heads)]
    assert sorted(units) == [(b, h) for b in range(4) for h in range(6)]


def test_slices_are_views_of_the_right_heads():
    q = torch.arange(2 * 8 * 3 * 4).reshape(2, 8, 3, 4)
    k = torch.arange(2 * 4 * 3 * 4).reshape(2, 4, 3, 4)
    s = P.prefill_shard(2, 4, 4, 2)
    qs, ks, vs = P.slice_prefill(q, k, k, s)
    assert torch.equal(qs, q[:, 4:6]) and torch.equal(ks, k[:, 2:3])
    assert qs.data_ptr() == q[:, 4:6].data_ptr()


def test_lpt_partition_balances_ragged_lengths():
    lens = W.decode_lengths(W.WORKLOADS["qwen3_8b_decode"])
    for world in (1, 2, 4, 8):
        parts = P.lpt_partition(lens, world)
        assert sorted(i for p in parts for i in p) == list(range(len(lens)))
        loads = [sum(lens[i] for i in p) for p in parts]
        assert max(loads) - min(loads) <= max(lens)
        assert max(loads) <= sum(lens) / world * 1.05 + 1
    assert P.lpt_partition([], 3) == [[], [], []]
    assert P.lpt_partition([5], 2) == [[0], []]


_RANK_SCRIPT = textwrap.dedent("""
    import os, sys, torch
    import torch.distributed as dist
    sys.path.insert(0, {root!r})
    from tyr_b200 import partition as P
    dist.init_process_group("gloo", rank=int(os.environ["RANK"]), world_size=2)
    rank = dist.get_rank()
    full = torch.arange(2 * 4 * 3 * 8, dtype=torch.float32).reshape(2, 4, 3, 8)
    for axis in ("heads", "batch"):
        if axis == "heads":
            shard = full[:, rank * 2:(rank + 1) * 2]
        else:
            shard = full[rank:rank + 1]
        got = P.gather_output(shard, axis)
        assert torch.equal(got, full), axis
    # a rank only ever computes its own shard: shards from the rule tile the work
    s = P.prefill_shard(2, 2, 2, rank)
    assert s.kv_heads == (rank, rank + 1)
    dist.barrier()
    dist.destroy_process_group()
    print("rank", rank, "ok")
""")


def test_gather_output_two_ranks_gloo(tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(_RANK_SCRIPT.format(root=ROOT))
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    for p in procs:
        out, _ = p.communicate(timeout=120)
        assert p.returncode == 0, out
        assert "ok" in out
