#!/usr/bin/env python
"""Benchmark of the attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one attention forward over one batch of the workload.  Rank 0
prints ONE JSON line.  Default workload: the Qwen3-8B-shaped causal GQA prefill
(B=4, S=8192, 32/8 heads, D=128), the largest single-GPU prefill configuration.

At N > 1 that ONE workload is cut across the ranks by the shard rule of
tyr_b200/partition.py ((batch, KV-head group) units; one KV-head group per GPU
at 8): strong scaling, no collective on the data path, `value` = whole-job
causal-adjusted TFLOP/s from the max-over-ranks device time.  Every rank slices
its shard out of the same seeded global tensors and, outside the timed region,
checks rows of its own output against the CPU oracle at their GLOBAL indices;
the run exits non-zero on a miss.

Besides the contract keys the line carries the other workloads kernel-only under
"other_workloads" (N = 1) or "strong_scaling_sharded" (N > 1), decode as KV GB/s.

`--shard-of R/N` runs rank R's shard of the N-GPU job alone on one GPU, without a
process group: the shard's time and its oracle parity where N GPUs are not to be had.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from tyr_b200 import workloads as W  # noqa: E402

METRIC = "attention_tflops_causal_adjusted"
UNIT = "TFLOP/s"
DEFAULT_WORKLOAD = "qwen3_8b_prefill"
L2_BYTES = 126 << 20
O_MAX_ABS, LSE_REL = 2e-2, 1e-3        # the parity bars for bf16 I/O


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def load_ncu_traffic(workload: str):
    """DRAM bytes of one launch of the workload's dominant kernel, from the ncu capture whose
    summary sits under profiles/ (profiles/ncu_traffic.json names the capture); None if none."""
    path = os.path.join(ROOT, "profiles", "ncu_traffic.json")
    if not os.path.exists(path):
        return None, None
    with open(path) as f:
        table = json.load(f)
    ent = table.get(workload)
    if not ent:
        return None, None
    return ent.get("dram_bytes_per_launch"), ent.get("source")


class ClockSampler:
    """SM clock and throttle reasons (read-only NVML queries) while the GPU runs the steps."""
    BITS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
            "sw_power_cap": 0x4}

    def __init__(self, cuda_index: int):
        self.samples, self._stop, self.max_mhz, self._h = [], threading.Event(), None, None
        try:
            import pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(cuda_index).uuid)
            uuid = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
            try:
                self._h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self._h = pynvml.nvmlDeviceGetHandleByIndex(cuda_index)
            self._nv = pynvml
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._h = None
        self._t = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)
                try:
                    reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                except Exception:
                    reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                self.samples.append((float(mhz), int(reasons)))
            except Exception:
                pass
            self._stop.wait(0.004)

    def __enter__(self):
        if self._h is not None:
            self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._h is not None:
            self._t.join(timeout=10)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unsampled"]}
        reasons = [n for n, bit in self.BITS.items() if any(r & bit for _, r in self.samples)]
        return {"sm_mhz": statistics.median(m for m, _ in self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(self.samples),
                "window": "warm-up + timed steps + 0.6 s of the same launches"}


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))


def split_workspace(tnn, q, k, v, causal):
    """Scratch for the key-split of a half-empty last round, kept across steps (None: the call would not split)."""
    need = tnn.prefill_workspace_bytes(q, k, v, is_causal=causal)
    return torch.empty(need, dtype=torch.uint8, device=q.device) if need > 0 else None


def shard_of(w, world, rank):
    from tyr_b200 import partition as P
    return P.prefill_shard(w.batch, w.n_kv_head, world, rank)


def workload_config(w, world):
    sh = shard_of(w, world, 0)
    nb, nh = sh.batch[1] - sh.batch[0], sh.kv_heads[1] - sh.kv_heads[0]
    g = w.n_head // w.n_kv_head
    shard_bytes = (2 * nb * nh * g + 2 * nb * nh) * w.seq * w.head_dim * 2
    sets = rotation_sets(shard_bytes)
    return {"workload": w.name, "global_batch": w.batch, "n_head": w.n_head, "n_kv_head": w.n_kv_head,
            "seq_len": w.seq, "head_dim": w.head_dim, "causal": w.causal,
            "parallelism": (f"one workload cut into {world} shards of batch {nb} x {nh} KV-head group(s) "
                            f"(axis: {sh.axis}); no collective on the data path") if world > 1 else
                           "one GPU, whole workload",
            "l2": (f"shard of {shard_bytes >> 20} MB of Q/K/V/O per step: " +
                   ("larger than the 126 MB L2" if sets == 1 else
                    f"the timed steps rotate over {sets} separate buffer sets ({sets * shard_bytes >> 20} MB), "
                    "so no step finds its inputs in L2"))}


def rotation_sets(nbytes: int) -> int:
    """Buffer sets the timed steps rotate over so that inputs never sit in L2 from the step before:
    1 when one set is larger than L2, else enough sets to exceed twice L2."""
    if nbytes > L2_BYTES:
        return 1
    return int(-(-2 * L2_BYTES // max(nbytes, 1)))


# ----------------------------------------------------------------- reference arm
def cpu_attention_step(q32, k32, v32, causal):
    """Tyr's LibTorch attention on the host: the ATen operator behind
    lean_torch_sdpa_gqa, with its repeat_interleave inside the timed call."""
    from oracle import aten_path
    return aten_path.sdpa_gqa(q32, k32, v32, 0.0, causal, True)


def cpu_sample_batch(w):
    """Batch elements of one CPU step: a bounded sample of the workload (about half a second of
    host work per step for the long-sequence workloads), the whole batch for the small ones."""
    per_elem = w.flops / w.batch
    return max(1, min(w.batch, int(1.0e12 // per_elem)))


def time_cpu(w, steps, warmup, sample_batch=None):
    q, k, v = W.make_prefill(w, batch=sample_batch)
    q32, k32, v32 = q.float(), k.float(), v.float()    # fp32 from bf16-rounded values
    for _ in range(warmup):
        cpu_attention_step(q32, k32, v32, w.causal)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        cpu_attention_step(q32, k32, v32, w.causal)
        times.append(time.perf_counter() - t0)
    frac = (sample_batch or w.batch) / w.batch
    return w.flops * frac, times


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return 0
    w = W.WORKLOADS[args.workload]
    # torchrun exports OMP_NUM_THREADS=1; the reference gets every host core it can use
    torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    sb = cpu_sample_batch(w)
    flops, times = time_cpu(w, args.steps, args.warmup, sample_batch=sb)
    sec = sum(times) / len(times)
    val = flops / sec / 1e12
    threads = torch.get_num_threads()
    sample = (f"{sb} of the {w.batch} batch elements of {w.name} per step (every head, full sequence): ATen "
              f"scaled_dot_product_attention on fp32 CPU tensors (bf16-rounded values), repeat_interleave GQA "
              f"expansion inside the call, torch {torch.__version__}")
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(w, max(args.gpus, 1)),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "reference", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)
    return 0


# ------------------------------------------------------------------------ our arm
def time_events(fn, steps, warmup, barrier):
    """fn(i) is step i.  Device time of `steps` steps after `warmup`, seconds."""
    for i in range(warmup):
        fn(i)
    barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(warmup + i)
    e1.record()
    torch.cuda.synchronize()
    barrier()
    return e0.elapsed_time(e1) / 1e3


def per_launch_ms(fn, n):
    """Average duration of single launches, each bracketed by its own events."""
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
    torch.cuda.synchronize()
    for i, (a, b) in enumerate(evs):
        a.record()
        fn(i)
        b.record()
    torch.cuda.synchronize()
    return sum(a.elapsed_time(b) for a, b in evs) / n


class Parity:
    """Running record of the oracle checks of one bench run."""

    def __init__(self):
        self.ok, self.max_abs, self.max_lse_rel, self.rows, self.where = True, 0.0, 0.0, 0, []

    def row(self, o_row, lse_val, ref_o, ref_lse, tag):
        err = float(np.abs(o_row - ref_o).max())
        bad = not np.isfinite(o_row).all() or err > O_MAX_ABS
        self.max_abs = max(self.max_abs, err)
        if lse_val is not None:
            rel = abs(float(lse_val) - float(ref_lse)) / max(abs(float(ref_lse)), 1.0)
            self.max_lse_rel = max(self.max_lse_rel, rel)
            bad = bad or rel > LSE_REL
        self.rows += 1
        if bad:
            self.ok = False
            self.where.append(tag)

    def summary(self):
        out = {"ok": self.ok, "max_abs": self.max_abs, "max_lse_rel": self.max_lse_rel, "rows": self.rows,
               "checker": "oracle/attn_oracle.c (exact softmax(QK^T)V in double precision) on rows sampled "
                          "at their global (batch, head, row) indices",
               "bars": {"o_max_abs": O_MAX_ABS, "lse_rel": LSE_REL}}
        if self.where:
            out["failed"] = self.where[:8]
        return out


def check_rows(par, qg, kg, vg, causal, o, lse, b_off, h_off, n_rows, seed, tag):
    """Exact oracle rows for a sample of the output `o` [nb, nh, S, D] of a shard whose first
    element is global (batch b_off, query head h_off).  qg, kg, vg are the GLOBAL bf16 CPU
    tensors: the oracle never sees the slicing the device path went through.  A row needs only
    its own keys, so one row of an 8192-long sequence costs microseconds."""
    from oracle import c_oracle
    nb, nh, S, D = o.shape
    g = qg.shape[1] // kg.shape[1]
    rng = np.random.default_rng(seed)
    edge = [0, S - 1, 127, 128, 255, 256, S // 2]
    picks = []
    for j in range(n_rows):
        bl, hl, i = int(rng.integers(nb)), int(rng.integers(nh)), int(rng.integers(S))
        if j % 6 == 0:
            i = min(edge[(j // 6) % len(edge)], S - 1)
        picks.append((bl, hl, i))
    idx = torch.tensor(picks, dtype=torch.long, device=o.device)
    o_rows = o[idx[:, 0], idx[:, 1], idx[:, 2]].float().cpu().numpy()
    l_rows = lse[idx[:, 0], idx[:, 1], idx[:, 2]].cpu().numpy() if lse is not None else None
    for j, (bl, hl, i) in enumerate(picks):
        b, h = b_off + bl, h_off + hl
        n_keys = i + 1 if causal else kg.shape[2]
        ro, rl = c_oracle.sdpa(qg[b, h, i].float().numpy().reshape(1, 1, 1, D),
                               kg[b, h // g, :n_keys].float().numpy().reshape(1, 1, n_keys, D),
                               vg[b, h // g, :n_keys].float().numpy().reshape(1, 1, n_keys, D), False)
        par.row(o_rows[j], None if l_rows is None else l_rows[j], ro[0, 0, 0], rl[0, 0, 0], f"{tag}[b={b},h={h},row={i}]")


def check_decode(par, q, ks, vs, o, lse, tag):
    """Every sequence of a decode result against the oracle (q [n, Hq, D] bf16 on any device)."""
    from oracle import c_oracle
    qh, oh, lh = q.float().cpu().numpy(), o.float().cpu().numpy(), lse.cpu().numpy()
    n, Hq, D = qh.shape
    for b in range(n):
        ro, rl = c_oracle.sdpa(qh[b].reshape(1, Hq, 1, D), ks[b].float().cpu().numpy()[None],
                               vs[b].float().cpu().numpy()[None], False)
        for h in range(Hq):
            par.row(oh[b, h], lh[b, h], ro[0, h, 0], rl[0, h, 0], f"{tag}[seq={b},h={h}]")


def prefill_sets(w, sh, dev, pin_first=False):
    """The rank's shard of the seeded global workload, as `sets` identical buffer sets on the device.
    Returns (global CPU tensors, host shard tensors, list of (q, k, v, o, lse) device sets)."""
    from tyr_b200 import partition as P
    qg, kg, vg = W.make_prefill(w)
    qs, ks_, vs_ = (t.contiguous() for t in P.slice_prefill(qg, kg, vg, sh))
    if pin_first:
        qs, ks_, vs_ = qs.pin_memory(), ks_.pin_memory(), vs_.pin_memory()
    nbytes = (2 * qs.numel() + ks_.numel() + vs_.numel()) * 2
    sets = []
    for _ in range(rotation_sets(nbytes)):
        q, k, v = qs.to(dev), ks_.to(dev), vs_.to(dev)
        sets.append((q, k, v, torch.empty_like(q), torch.empty(q.shape[:3], dtype=torch.float32, device=dev)))
    return (qg, kg, vg), (qs, ks_, vs_), sets


def other_workloads(tnn, dev, peaks, par, steps=10, warmup=3):
    """The other four workloads, kernel-only, on the seeded inputs of tyr_b200/workloads.py, each
    with a sample of rows checked against the oracle after its timed region."""
    out = {}
    for name in ("qwen3_0p6b_prefill", "flux_mmdit", "gpt_char"):
        w = W.WORKLOADS[name]
        sh = shard_of(w, 1, 0)
        (qg, kg, vg), _, sets = prefill_sets(w, sh, dev)
        n = len(sets)

        ws = split_workspace(tnn, *sets[0][:3], w.causal)

        def step(i, sets=sets, n=n, w=w, ws=ws):
            q, k, v, o, lse = sets[i % n]
            tnn.attentionFwd(q, k, v, is_causal=w.causal, out=o, lse=lse, workspace=ws)
        sec = time_events(step, steps, warmup, lambda: None) / steps
        check_rows(par, qg, kg, vg, w.causal, sets[0][3], sets[0][4], 0, 0, 24, w.seed, name)
        out[name] = {"ms": sec * 1e3, "tflops": w.flops / sec / 1e12, "gbs": w.io_bytes / sec / 1e9,
                     "frac_tensor_peak": w.flops / sec / 1e12 / peaks["bf16_tflops"],
                     "frac_hbm_peak": w.io_bytes / sec / 1e9 / peaks["hbm_gbs"],
                     "buffer_sets": n}
        del sets, qg, kg, vg
    # backward of the two causal prefill workloads: row statistics + dK/dV + dQ kernels; FLOPs by the
    # usual convention of five score-sized products (2.5 x the forward)
    for name in ("qwen3_0p6b_prefill", "qwen3_8b_prefill"):
        w = W.WORKLOADS[name]
        q, k, v = (t.to(dev) for t in W.make_prefill(w))
        g = torch.Generator(device=dev).manual_seed(w.seed + 100)
        d_o = torch.randn(q.shape, device=dev, generator=g).bfloat16()
        o, lse = tnn.attentionFwd(q, k, v, is_causal=w.causal)
        ws = torch.empty(2 * lse.numel(), device=dev)
        sec = time_events(lambda i: tnn.attentionBwd(q, k, v, o, lse, d_o, is_causal=w.causal, workspace=ws),
                          steps, warmup, lambda: None) / steps
        out[name.replace("prefill", "backward")] = {
            "ms": sec * 1e3, "tflops": 2.5 * w.flops / sec / 1e12,
            "frac_tensor_peak": 2.5 * w.flops / sec / 1e12 / peaks["bf16_tflops"],
            "note": "7 score-sized products are executed (S and dP are recomputed by the dQ kernel); 5 are counted"}
        del q, k, v, d_o, o, lse, ws
    w = W.WORKLOADS["qwen3_8b_decode"]
    q, ks, vs, lens = W.make_decode(w, device=str(dev))   # seeded lengths and values, drawn on the device
    q = q.to(dev)
    plan = tnn.DecodePlan(ks, vs, w.n_head)
    o, lse = torch.empty_like(q), torch.empty(q.shape[:2], device=dev)
    sec = time_events(lambda i: tnn.flashDecode(q, plan, out=o, lse=lse), steps, warmup, lambda: None) / steps
    check_decode(par, q[:8], ks[:8], vs[:8], o[:8], lse[:8], w.name)
    byts = W.decode_kv_bytes(lens, w.n_kv_head, w.head_dim)
    out[w.name] = {"ms": sec * 1e3, "kv_gbs": byts / sec / 1e9, "kv_bytes": byts,
                   "frac_hbm_peak": byts / sec / 1e9 / peaks["hbm_gbs"],
                   "l2": "4.8 GB of KV per step, far above L2"}
    del plan, ks, vs
    # fused K prologue (RMSNorm + rotary + layout + append): 4096 new tokens per sequence appended
    # to a dense cache; bytes = one read + one write
    B, S, H, D, cap = 16, 4096, 8, 128, 8192
    g = torch.Generator(device=dev).manual_seed(5)
    x = torch.randn(B, S, H, D, device=dev, generator=g).bfloat16()
    cache = torch.zeros(B, H, cap, D, device=dev, dtype=torch.bfloat16)
    wn = torch.ones(D, device=dev)
    ang = torch.arange(cap, device=dev).float()[:, None] * (1.0 / (10000.0 ** (torch.arange(D // 2, device=dev).float() / (D // 2))))[None]
    cs, sn = ang.cos().contiguous(), ang.sin().contiguous()
    pos = torch.full((B,), 1024, dtype=torch.int32, device=dev)
    sec = time_events(lambda i: tnn.qkPrologue(x, cache, wn, cs, sn, positions=pos), steps, warmup, lambda: None) / steps
    byts = 2 * x.numel() * 2
    out["k_prologue_append"] = {"ms": sec * 1e3, "gbs": byts / sec / 1e9, "bytes": byts,
                                "frac_hbm_peak": byts / sec / 1e9 / peaks["hbm_gbs"],
                                "l2": "134 MB in + 134 MB out per step, above L2"}
    return out


def sharded_workloads(tnn, dev, rank, world, barrier, all_max, par, steps=10, warmup=3):
    """Strong scaling of the other shardable workloads at N > 1: ONE seeded workload cut across the
    ranks by the shard rules of tyr_b200/partition.py (KV-head groups, else batch; LPT split for
    decode), no collective on the data path.  Time = max over ranks of the device time; value =
    whole-job work / time.  Every rank checks its own shard against the oracle afterwards."""
    from tyr_b200 import partition as P
    out = {}
    w = W.WORKLOADS["flux_mmdit"]
    sh = P.prefill_shard(w.batch, w.n_kv_head, world, rank)
    g_ = w.n_head // w.n_kv_head
    (qg, kg, vg), _, sets = prefill_sets(w, sh, dev)
    n = len(sets)

    ws = split_workspace(tnn, *sets[0][:3], w.causal)

    def step(i):
        q, k, v, o, lse = sets[i % n]
        tnn.attentionFwd(q, k, v, is_causal=w.causal, out=o, lse=lse, workspace=ws)
    sec = all_max(time_events(step, steps, warmup, barrier) / steps)
    check_rows(par, qg, kg, vg, w.causal, sets[0][3], sets[0][4], sh.batch[0], sh.kv_heads[0] * g_, 16,
               w.seed + rank, f"{w.name}@rank{rank}")
    nb, nh = sh.batch[1] - sh.batch[0], sh.kv_heads[1] - sh.kv_heads[0]
    out[w.name] = {"ms": sec * 1e3, "tflops": w.flops / sec / 1e12, "shard_axis": sh.axis,
                   "shard": f"batch {nb} x kv_heads {nh} per GPU", "buffer_sets": n,
                   "last_round_key_split": ws is not None}
    del sets, qg, kg, vg

    w = W.WORKLOADS["qwen3_8b_decode"]
    # the one seeded workload, drawn identically on every rank's device; a rank keeps its own sequences
    q_all, ks_all, vs_all, lens = W.make_decode(w, device=str(dev))
    mine = P.lpt_partition(lens, world)[rank]
    ks = [ks_all[i] for i in mine]
    vs = [vs_all[i] for i in mine]
    q = q_all[mine].to(dev)
    del ks_all, vs_all
    torch.cuda.empty_cache()
    plan = tnn.DecodePlan(ks, vs, w.n_head)
    o, lse = torch.empty_like(q), torch.empty(q.shape[:2], device=dev)
    sec = all_max(time_events(lambda i: tnn.flashDecode(q, plan, out=o, lse=lse), steps, warmup, barrier) / steps)
    check_decode(par, q, ks, vs, o, lse, f"{w.name}@rank{rank}")
    byts = W.decode_kv_bytes(lens, w.n_kv_head, w.head_dim)
    out[w.name] = {"ms": sec * 1e3, "kv_gbs": byts / sec / 1e9, "shard": "sequences by greedy length-balanced split",
                   "sequences_on_rank0": len(mine),
                   "l2": f"{W.decode_kv_bytes([lens[i] for i in mine], w.n_kv_head, w.head_dim) >> 20} MB of KV per rank per step, above L2"}
    return out


def run_profile(args):
    """warm-up + steps launches of one kernel and nothing else (for ncu captures)."""
    from tyr_b200 import nn as tnn
    dev = torch.device("cuda", 0)
    if args.profile == "prefill":
        from tyr_b200 import partition as P
        w = W.WORKLOADS[args.workload]
        r_, n_ = (int(x) for x in args.shard_of.split("/")) if args.shard_of else (0, 1)   # one shard of an N-way cut
        q, k, v = (t.contiguous().to(dev) for t in P.slice_prefill(*W.make_prefill(w), P.prefill_shard(w.batch, w.n_kv_head, n_, r_)))
        o, lse = torch.empty_like(q), torch.empty(q.shape[:3], dtype=torch.float32, device=dev)
        ws = split_workspace(tnn, q, k, v, w.causal)
        step = lambda i: tnn.attentionFwd(q, k, v, is_causal=w.causal, out=o, lse=lse, workspace=ws)  # noqa: E731
        work, unit = w.flops / n_ / 1e12, "TFLOP/s"
    elif args.profile == "backward":
        w = W.WORKLOADS[args.workload]
        q, k, v = (t.to(dev) for t in W.make_prefill(w))
        g = torch.Generator(device=dev).manual_seed(w.seed + 100)
        d_o = torch.randn(q.shape, device=dev, generator=g).bfloat16()
        o, lse = tnn.attentionFwd(q, k, v, is_causal=w.causal)
        ws = torch.empty(2 * lse.numel(), device=dev)
        step = lambda i: tnn.attentionBwd(q, k, v, o, lse, d_o, is_causal=w.causal, workspace=ws)  # noqa: E731
        work, unit = 2.5 * w.flops / 1e12, "TFLOP/s"
    elif args.profile == "prologue":
        w = W.WORKLOADS["qwen3_8b_decode"]
        B, S, H, D, cap = 16, 4096, 8, 128, 8192
        g = torch.Generator(device=dev).manual_seed(5)
        x = torch.randn(B, S, H, D, device=dev, generator=g).bfloat16()
        cache = torch.zeros(B, H, cap, D, device=dev, dtype=torch.bfloat16)
        wn = torch.ones(D, device=dev)
        ang = torch.arange(cap, device=dev).float()[:, None] * (1.0 / (10000.0 ** (torch.arange(D // 2, device=dev).float() / (D // 2))))[None]
        cs, sn = ang.cos().contiguous(), ang.sin().contiguous()
        pos = torch.full((B,), 1024, dtype=torch.int32, device=dev)
        step = lambda i: tnn.qkPrologue(x, cache, wn, cs, sn, positions=pos)  # noqa: E731
        work, unit = 2 * x.numel() * 2 / 1e9, "GB/s"
    else:
        w = W.WORKLOADS["qwen3_8b_decode"]
        q, ks, vs, lens = W.make_decode(w, batch=args.decode_batch, device=str(dev))
        q = q.to(dev)
        plan = tnn.DecodePlan(ks, vs, w.n_head)
        o, lse = torch.empty_like(q), torch.empty(q.shape[:2], dtype=torch.float32, device=dev)
        step = lambda i: tnn.flashDecode(q, plan, out=o, lse=lse)  # noqa: E731
        work, unit = W.decode_kv_bytes(lens, w.n_kv_head, w.head_dim) / 1e9, "GB/s"
    sec = time_events(step, args.steps, args.warmup, lambda: None) / args.steps
    status = tnn.device_status(0, True)
    print(json.dumps({"profile": args.profile, "workload": w.name, "ms_per_step": sec * 1e3,
                      "value": work / sec, "unit": unit, "steps": args.steps, "warmup": args.warmup,
                      "device_status": status}), flush=True)
    return 0 if status == 0 else 1


def run_ours(args):
    from tyr_b200 import nn as tnn
    from tyr_b200 import partition as P
    rank, world, local = dist_env()
    world = max(world, 1)
    solo = args.shard_of is not None
    if solo:  # one rank's shard of an N-way job, alone on one GPU and without a process group
        rank, world = (int(x) for x in args.shard_of.split("/"))
        assert 0 <= rank < world
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    use_dist = world > 1 and not solo
    if use_dist:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        barrier = lambda: dist.barrier()  # noqa: E731
    else:
        barrier = lambda: None  # noqa: E731

    def all_max(x):
        tt = torch.tensor([x], dtype=torch.float64, device=dev)
        if use_dist:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item())

    def all_and(flag):
        tt = torch.tensor([1.0 if flag else 0.0], dtype=torch.float64, device=dev)
        if use_dist:
            dist.all_reduce(tt, op=dist.ReduceOp.MIN)
        return bool(tt.item() > 0.5)

    peaks = load_peaks()
    w = W.WORKLOADS[args.workload]
    assert w.kind == "prefill", "the headline bench line is a prefill workload"
    sh = P.prefill_shard(w.batch, w.n_kv_head, world, rank)
    g_ = w.n_head // w.n_kv_head
    (qg, kg, vg), (qh, kh, vh), sets = prefill_sets(w, sh, dev, pin_first=True)
    n_sets = len(sets)

    ws = split_workspace(tnn, *sets[0][:3], w.causal)

    def step(i):
        q, k, v, o, lse = sets[i % n_sets]
        tnn.attentionFwd(q, k, v, is_causal=w.causal, out=o, lse=lse, workspace=ws)

    n0 = tnn.launch_count()
    with ClockSampler(local) as clocks:
        total = time_events(step, args.steps, args.warmup, barrier)
        # keep the GPU under the same load while the sampler collects enough points
        t_end = time.perf_counter() + 0.6
        i = 0
        while time.perf_counter() < t_end:
            for _ in range(20):
                step(i)
                i += 1
            torch.cuda.synchronize()
    launches = args.steps * (2 if ws is not None else 1)   # a split launch is the kernel and its merge
    assert tnn.launch_count() - n0 >= args.steps + args.warmup
    if tnn.device_status(local, True) != 0:
        raise RuntimeError("a bounded in-kernel wait gave up during the benchmark")
    total = all_max(total)
    sec = total / args.steps
    value = w.flops / sec / 1e12          # the WHOLE workload over the slowest rank's time

    # parity of this rank's shard, outside the timed region: oracle rows at their global indices
    par = Parity()
    step(0)
    torch.cuda.synchronize()
    check_rows(par, qg, kg, vg, w.causal, sets[0][3], sets[0][4], sh.batch[0], sh.kv_heads[0] * g_,
               48 if world == 1 else 24, w.seed + 17 * rank, f"{w.name}@rank{rank}")
    gather_ms = None
    if use_dist and sh.axis in ("heads", "batch"):
        # optional replicated output (only when a caller asks for it): one NCCL all-gather of the O
        # shards into local staging + a local permute; timed apart from the kernel, and the gathered
        # tensor is checked on rank 0 at global indices that fall into every rank's shard
        o_sh = sets[0][3]
        full = P.gather_output(o_sh, sh.axis)
        gsec = all_max(time_events(lambda i: P.gather_output(o_sh, sh.axis), 5, 2, barrier) / 5)
        gather_ms = gsec * 1e3
        if rank == 0:
            check_rows(par, qg, kg, vg, w.causal, full, None, 0, 0, 4 * world, w.seed + 999, f"{w.name}@gathered")
        del full

    # The timed region holds exactly one kernel, launched once per step, so its average launch
    # duration is the region's CUDA-event time over the steps (gaps between launches included).
    launch_ms = sec * 1e3
    launch_ms_bracketed = all_max(per_launch_ms(step, max(min(args.steps, 50), 20)))
    shard_flops = w.flops / world          # the shard rule gives every rank the same number of (batch, head) units
    achieved = shard_flops / (launch_ms / 1e3) / 1e12        # per-GPU: the slowest rank's shard over its time
    traffic, traffic_src = load_ncu_traffic(w.name) if world == 1 else (None, None)

    # end to end through the C ABI's host-buffer call: pinned host tensors in, host tensors out
    oh = torch.empty(qh.shape, dtype=torch.bfloat16).pin_memory()
    lseh = torch.empty(qh.shape[:3], dtype=torch.float32).pin_memory()
    for _ in range(2):
        tnn.sdpa_host(qh, kh, vh, is_causal=w.causal, out=oh, lse=lseh, device=local)
    barrier()
    t0 = time.perf_counter()
    e2e_steps = min(args.steps, 10)
    for _ in range(e2e_steps):
        tnn.sdpa_host(qh, kh, vh, is_causal=w.causal, out=oh, lse=lseh, device=local)
    e2e_sec = all_max((time.perf_counter() - t0) / e2e_steps)
    h2d = (qh.numel() + kh.numel() + vh.numel()) * 2
    d2h = oh.numel() * 2 + lseh.numel() * 4
    # the host-buffer call's result gets the same oracle rows
    check_rows(par, qg, kg, vg, w.causal, oh, lseh, sh.batch[0], sh.kv_heads[0] * g_, 8, w.seed + 5, f"{w.name}@host-call")

    sharded = None
    if (use_dist or solo) and not args.no_others:
        del sets
        sharded = sharded_workloads(tnn, dev, rank, world, barrier, all_max, par)

    cpu, others = None, None
    if world == 1 and rank == 0:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
        sb = cpu_sample_batch(w)
        flops, times = time_cpu(w, 3, 1, sample_batch=sb)
        best = min(times)
        cpu = {"value": flops / best / 1e12, "unit": UNIT, "cores": torch.get_num_threads(),
               "kind": "reference",
               "sample": (f"{sb} of the {w.batch} batch elements of {w.name}, best of 3: ATen scaled_dot_product_attention "
                          f"(the call at cc/src/tyr.cpp:3941) on fp32 CPU tensors via torch {torch.__version__}, "
                          "repeat_interleave inside the timed call"),
               "ms": best * 1e3, "host_cpus": os.cpu_count()}
        if not args.no_others:
            del sets
            others = other_workloads(tnn, dev, peaks, par)

    parity_ok = all_and(par.ok)
    rows_total = par.rows
    if use_dist:
        tt = torch.tensor([float(par.rows), par.max_abs, par.max_lse_rel], dtype=torch.float64, device=dev)
        rows_t = tt[:1].clone()
        dist.all_reduce(rows_t, op=dist.ReduceOp.SUM)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        rows_total, par.max_abs, par.max_lse_rel = int(rows_t.item()), float(tt[1].item()), float(tt[2].item())
    if not par.ok:
        print(f"rank {rank}: PARITY MISS {par.where[:8]}", file=sys.stderr, flush=True)

    if rank == 0 or solo:
        psum = par.summary()
        psum["ok"], psum["rows"] = parity_ok, rows_total
        psum["ranks_checked"] = world
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(w, world),
            "clocks": clocks.summary(),
            "e2e": {"value": w.flops / e2e_sec / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d * world,
                    "d2h_bytes_per_step": d2h * world, "ms_per_step": e2e_sec * 1e3,
                    "api": "tyr_b200_attn_prefill_host on each rank's shard (pinned host buffers; bytes are "
                           "the whole job's)"},
            "gpu_launches": launches,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"],
                         "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"], "traffic": traffic,
                         "traffic_source": traffic_src,
                         "kernel": "prefill_kernel<128>: the slowest rank's shard FLOPs over its launch time",
                         "peak_source": peaks["source"] + " bf16_tflops (burst: kernel timed alone)",
                         "launch_ms": launch_ms, "launch_ms_bracketed": launch_ms_bracketed,
                         "algorithmic_flops_per_launch": shard_flops,
                         "frac_of_sustained": (achieved / peaks["bf16_tflops_sustained"]
                                               if peaks.get("bf16_tflops_sustained") else None),
                         "frac_of_nominal_2250": achieved / 2250.0},
            "cpu_baseline": cpu,
            "parity": psum,
        }
        if gather_ms is not None:
            line["replicate_output"] = {"ms": gather_ms, "gbs_per_gpu": sets_bytes_o(w, sh) * (world - 1) / (gather_ms / 1e3) / 1e9,
                                        "note": "optional NCCL all-gather of the O shards + local permute; not part of the metric"}
        if others is not None:
            line["other_workloads"] = others
        if sharded is not None:
            line["strong_scaling_sharded"] = sharded
        if solo:
            line["shard_of"] = {"rank": rank, "world": world,
                                "note": "this rank's shard alone on one GPU: value = whole-job work over this shard's time"}
            line["parity"]["ranks_checked"] = 1
        print(json.dumps(line), flush=True)
    if use_dist:
        dist.barrier()
        dist.destroy_process_group()
    return 0 if parity_ok else 3


def sets_bytes_o(w, sh):
    nb, nh = sh.batch[1] - sh.batch[0], sh.kv_heads[1] - sh.kv_heads[0]
    return nb * nh * (w.n_head // w.n_kv_head) * w.seq * w.head_dim * 2


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=[n for n, w in W.WORKLOADS.items() if w.kind == "prefill"])
    ap.add_argument("--no-others", action="store_true", help="skip the extra kernel-only workloads")
    ap.add_argument("--shard-of", default=None, metavar="R/N",
                    help="run rank R's shard of an N-GPU job alone on one GPU (no process group): its time and parity")
    ap.add_argument("--profile", choices=["prefill", "backward", "decode", "prologue"], default=None,
                    help="profiler-friendly run: only warm-up + steps of one kernel, no e2e/CPU legs")
    ap.add_argument("--decode-batch", type=int, default=None, help="sequences of the decode workload (profile runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return run_reference(args)
    if args.profile:
        return run_profile(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
