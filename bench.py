#!/usr/bin/env python
"""Benchmark of the attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one attention forward over one batch of the workload.  Rank 0
prints ONE JSON line.  Default workload: the Qwen3-0.6B-shaped causal GQA
prefill (B=8, S=2048, 16/8 heads, D=128).  At N > 1 every rank runs that same
batch on its own GPU (weak scaling: the units are independent, no collective on
the data path) and `value` is the whole-job throughput.

Besides the contract keys the line carries the other four workloads measured
kernel-only under "other_workloads" (decode as KV GB/s).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from tyr_b200 import workloads as W  # noqa: E402

METRIC = "attention_tflops_causal_adjusted"
UNIT = "TFLOP/s"
DEFAULT_WORKLOAD = "qwen3_0p6b_prefill"
# dram__bytes_read.sum + dram__bytes_write.sum of one prefill launch, from the ncu
# capture summarised in profiles/prefill_kernel_qwen3_0p6b_prefill.md (None: no capture for that workload)
NCU_TRAFFIC_BYTES = {"qwen3_0p6b_prefill": 258017024}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


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


# ----------------------------------------------------------------- reference arm
def cpu_attention_step(q32, k32, v32, causal):
    """Tyr's LibTorch attention on the host: the ATen operator behind
    lean_torch_sdpa_gqa, with its repeat_interleave inside the timed call."""
    from oracle import aten_path
    return aten_path.sdpa_gqa(q32, k32, v32, 0.0, causal, True)


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
    flops = w.flops * frac
    return flops, times


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return 0
    w = W.WORKLOADS[args.workload]
    # torchrun exports OMP_NUM_THREADS=1; the reference gets every host core it can use
    torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    flops, times = time_cpu(w, args.steps, args.warmup)
    sec = sum(times) / len(times)
    val = flops / sec / 1e12
    threads = torch.get_num_threads()
    sample = (f"one GPU's {w.name} batch (B={w.batch}) per step: ATen scaled_dot_product_attention on fp32 CPU tensors "
              f"(bf16-rounded values), repeat_interleave GQA expansion inside the call, torch {torch.__version__}")
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(w, max(args.gpus, 1)),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "reference", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)
    return 0


def workload_config(w, world):
    return {"workload": w.name, "batch_per_gpu": w.batch, "global_batch": w.batch * world,
            "n_head": w.n_head, "n_kv_head": w.n_kv_head, "seq_len": w.seq, "head_dim": w.head_dim,
            "causal": w.causal, "parallelism": f"replicated-units x{world} (no collective)",
            "l2": "inputs larger than L2 (202 MB of Q/K/V/O per step vs 126 MB)"}


# ------------------------------------------------------------------------ our arm
def time_events(fn, steps, warmup, barrier):
    for _ in range(warmup):
        fn()
    barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    barrier()
    return e0.elapsed_time(e1) / 1e3   # seconds for all steps


def per_launch_ms(fn, n):
    """Average duration of single launches, each bracketed by its own events."""
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
    torch.cuda.synchronize()
    for a, b in evs:
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    return sum(a.elapsed_time(b) for a, b in evs) / n


def other_workloads(tnn, dev, peaks, steps=10, warmup=3):
    out = {}
    for name in ("gpt_char", "qwen3_8b_prefill", "flux_mmdit"):
        w = W.WORKLOADS[name]
        g = torch.Generator(device=dev).manual_seed(w.seed)
        q = torch.randn(w.batch, w.n_head, w.seq, w.head_dim, device=dev, generator=g).bfloat16()
        k = torch.randn(w.batch, w.n_kv_head, w.seq, w.head_dim, device=dev, generator=g).bfloat16()
        v = torch.randn(w.batch, w.n_kv_head, w.seq, w.head_dim, device=dev, generator=g).bfloat16()
        o, lse = torch.empty_like(q), torch.empty(q.shape[:3], device=dev)
        sec = time_events(lambda: tnn.attentionFwd(q, k, v, is_causal=w.causal, out=o, lse=lse), steps, warmup,
                          lambda: None) / steps
        out[name] = {"ms": sec * 1e3, "tflops": w.flops / sec / 1e12, "gbs": w.io_bytes / sec / 1e9,
                     "frac_tensor_peak": w.flops / sec / 1e12 / peaks["bf16_tflops"],
                     "frac_hbm_peak": w.io_bytes / sec / 1e9 / peaks["hbm_gbs"]}
        del q, k, v, o, lse
    # backward of the headline and of the long-sequence workload: row statistics + dK/dV + dQ
    # kernels; FLOPs by the usual convention of five score-sized products (2.5 x the forward)
    for name in ("qwen3_0p6b_prefill", "qwen3_8b_prefill"):
        w = W.WORKLOADS[name]
        g = torch.Generator(device=dev).manual_seed(w.seed)
        q = torch.randn(w.batch, w.n_head, w.seq, w.head_dim, device=dev, generator=g).bfloat16()
        k = torch.randn(w.batch, w.n_kv_head, w.seq, w.head_dim, device=dev, generator=g).bfloat16()
        v = torch.randn(w.batch, w.n_kv_head, w.seq, w.head_dim, device=dev, generator=g).bfloat16()
        d_o = torch.randn(w.batch, w.n_head, w.seq, w.head_dim, device=dev, generator=g).bfloat16()
        o, lse = tnn.attentionFwd(q, k, v, is_causal=w.causal)
        ws = torch.empty(2 * lse.numel(), device=dev)
        sec = time_events(lambda: tnn.attentionBwd(q, k, v, o, lse, d_o, is_causal=w.causal, workspace=ws),
                          steps, warmup, lambda: None) / steps
        out[name.replace("prefill", "backward")] = {
            "ms": sec * 1e3, "tflops": 2.5 * w.flops / sec / 1e12,
            "frac_tensor_peak": 2.5 * w.flops / sec / 1e12 / peaks["bf16_tflops"],
            "note": "7 score-sized products are executed (S and dP are recomputed by the dQ kernel); 5 are counted"}
        del q, k, v, d_o, o, lse, ws
    w = W.WORKLOADS["qwen3_8b_decode"]
    q, ks, vs, lens = W.make_decode(w, device=str(dev))
    q = q.to(dev)
    plan = tnn.DecodePlan(ks, vs, w.n_head)
    o, lse = torch.empty_like(q), torch.empty(q.shape[:2], device=dev)
    sec = time_events(lambda: tnn.flashDecode(q, plan, out=o, lse=lse), steps, warmup, lambda: None) / steps
    byts = W.decode_kv_bytes(lens, w.n_kv_head, w.head_dim)
    out[w.name] = {"ms": sec * 1e3, "kv_gbs": byts / sec / 1e9, "kv_bytes": byts,
                   "frac_hbm_peak": byts / sec / 1e9 / peaks["hbm_gbs"],
                   "l2": "4.8 GB of KV per step, far above L2"}
    # fused K prologue (RMSNorm + rotary + layout + append) on the decode workload's batch:
    # 4096 new tokens per sequence appended to a dense cache; bytes = one read + one write
    B, S, H, D, cap = 16, 4096, 8, 128, 8192
    g = torch.Generator(device=dev).manual_seed(5)
    x = torch.randn(B, S, H, D, device=dev, generator=g).bfloat16()
    cache = torch.zeros(B, H, cap, D, device=dev, dtype=torch.bfloat16)
    wn = torch.ones(D, device=dev)
    ang = torch.arange(cap, device=dev).float()[:, None] * (1.0 / (10000.0 ** (torch.arange(D // 2, device=dev).float() / (D // 2))))[None]
    cs, sn = ang.cos().contiguous(), ang.sin().contiguous()
    pos = torch.full((B,), 1024, dtype=torch.int32, device=dev)
    sec = time_events(lambda: tnn.qkPrologue(x, cache, wn, cs, sn, positions=pos), steps, warmup, lambda: None) / steps
    byts = 2 * x.numel() * 2
    out["k_prologue_append"] = {"ms": sec * 1e3, "gbs": byts / sec / 1e9, "bytes": byts,
                                "frac_hbm_peak": byts / sec / 1e9 / peaks["hbm_gbs"],
                                "l2": "134 MB in + 134 MB out per step, above L2"}
    return out


def sharded_workloads(tnn, dev, rank, world, barrier, all_max, steps=10, warmup=3):
    """Strong scaling at N > 1: ONE fixed workload cut across the ranks by the shard rules of
    tyr_b200/partition.py (KV-head groups, else batch; LPT split for decode), no collective on
    the data path.  Time = max over ranks of the device time; value = whole-job work / time."""
    from tyr_b200 import partition as P
    out = {}
    for name in ("qwen3_8b_prefill", "flux_mmdit"):
        w = W.WORKLOADS[name]
        sh = P.prefill_shard(w.batch, w.n_kv_head, world, rank)
        g_ = w.n_head // w.n_kv_head
        nb, nh = sh.batch[1] - sh.batch[0], sh.kv_heads[1] - sh.kv_heads[0]
        gen = torch.Generator(device=dev).manual_seed(w.seed + rank)
        q = torch.randn(nb, nh * g_, w.seq, w.head_dim, device=dev, generator=gen).bfloat16()
        k = torch.randn(nb, nh, w.seq, w.head_dim, device=dev, generator=gen).bfloat16()
        v = torch.randn(nb, nh, w.seq, w.head_dim, device=dev, generator=gen).bfloat16()
        o, lse = torch.empty_like(q), torch.empty(q.shape[:3], device=dev)
        sec = all_max(time_events(lambda: tnn.attentionFwd(q, k, v, is_causal=w.causal, out=o, lse=lse),
                                  steps, warmup, barrier) / steps)
        out[name] = {"ms": sec * 1e3, "tflops": w.flops / sec / 1e12, "shard_axis": sh.axis,
                     "shard": f"batch {nb} x kv_heads {nh} per GPU"}
        if sh.axis in ("heads", "batch"):
            # optional replicated output (only when a caller asks for it): one NCCL all-gather of
            # the O shards into local staging + a local permute; reported apart from the kernel
            gsec = all_max(time_events(lambda: P.gather_output(o, sh.axis), 5, 2, barrier) / 5)
            out[name]["replicate_output_ms"] = gsec * 1e3
            out[name]["replicate_output_gbs_per_gpu"] = o.numel() * 2 * (world - 1) / gsec / 1e9
        del q, k, v, o, lse
    w = W.WORKLOADS["qwen3_8b_decode"]
    lens = W.decode_lengths(w)
    mine = P.lpt_partition(lens, world)[rank]
    gen = torch.Generator(device=dev).manual_seed(w.seed + rank)
    ks = [torch.randn(w.n_kv_head, lens[i], w.head_dim, device=dev, generator=gen).bfloat16() for i in mine]
    vs = [torch.randn(w.n_kv_head, lens[i], w.head_dim, device=dev, generator=gen).bfloat16() for i in mine]
    q = torch.randn(len(mine), w.n_head, w.head_dim, device=dev, generator=gen).bfloat16()
    plan = tnn.DecodePlan(ks, vs, w.n_head)
    o, lse = torch.empty_like(q), torch.empty(q.shape[:2], device=dev)
    sec = all_max(time_events(lambda: tnn.flashDecode(q, plan, out=o, lse=lse), steps, warmup, barrier) / steps)
    byts = W.decode_kv_bytes(lens, w.n_kv_head, w.head_dim)
    out[w.name] = {"ms": sec * 1e3, "kv_gbs": byts / sec / 1e9, "shard": "sequences by greedy length-balanced split",
                   "sequences_on_rank0": len(mine)}
    return out


def run_profile(args):
    """warm-up + steps launches of one kernel and nothing else (for ncu captures)."""
    from tyr_b200 import nn as tnn
    dev = torch.device("cuda", 0)
    if args.profile == "prefill":
        w = W.WORKLOADS[args.workload]
        q, k, v = (t.to(dev) for t in W.make_prefill(w))
        o, lse = torch.empty_like(q), torch.empty(q.shape[:3], dtype=torch.float32, device=dev)
        step = lambda: tnn.attentionFwd(q, k, v, is_causal=w.causal, out=o, lse=lse)  # noqa: E731
        work, unit = w.flops / 1e12, "TFLOP/s"
    elif args.profile == "backward":
        w = W.WORKLOADS[args.workload]
        q, k, v = (t.to(dev) for t in W.make_prefill(w))
        g = torch.Generator(device=dev).manual_seed(w.seed + 100)
        d_o = torch.randn(q.shape, device=dev, generator=g).bfloat16()
        o, lse = tnn.attentionFwd(q, k, v, is_causal=w.causal)
        ws = torch.empty(2 * lse.numel(), device=dev)
        step = lambda: tnn.attentionBwd(q, k, v, o, lse, d_o, is_causal=w.causal, workspace=ws)  # noqa: E731
        work, unit = 2.5 * w.flops / 1e12, "TFLOP/s"
    else:
        w = W.WORKLOADS["qwen3_8b_decode"]
        q, ks, vs, lens = W.make_decode(w, batch=args.decode_batch, device=str(dev))
        q = q.to(dev)
        plan = tnn.DecodePlan(ks, vs, w.n_head)
        o, lse = torch.empty_like(q), torch.empty(q.shape[:2], dtype=torch.float32, device=dev)
        step = lambda: tnn.flashDecode(q, plan, out=o, lse=lse)  # noqa: E731
        work, unit = W.decode_kv_bytes(lens, w.n_kv_head, w.head_dim) / 1e9, "GB/s"
    sec = time_events(step, args.steps, args.warmup, lambda: None) / args.steps
    status = tnn.device_status(0, True)
    print(json.dumps({"profile": args.profile, "workload": w.name, "ms_per_step": sec * 1e3,
                      "value": work / sec, "unit": unit, "steps": args.steps, "warmup": args.warmup,
                      "device_status": status}), flush=True)
    return 0 if status == 0 else 1


def run_ours(args):
    from tyr_b200 import nn as tnn
    rank, world, local = dist_env()
    if world != args.gpus:
        world = max(world, 1)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    use_dist = world > 1
    if use_dist:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        barrier = lambda: dist.barrier()  # noqa: E731
    else:
        barrier = lambda: None  # noqa: E731
    peaks = load_peaks()
    w = W.WORKLOADS[args.workload]
    assert w.kind == "prefill", "the headline bench line is a prefill workload"

    qh, kh, vh = (t.pin_memory() for t in W.make_prefill(w))
    q, k, v = qh.to(dev), kh.to(dev), vh.to(dev)
    o = torch.empty_like(q)
    lse = torch.empty(q.shape[:3], dtype=torch.float32, device=dev)
    step = lambda: tnn.attentionFwd(q, k, v, is_causal=w.causal, out=o, lse=lse)  # noqa: E731

    n0 = tnn.launch_count()
    with ClockSampler(local) as clocks:
        total = time_events(step, args.steps, args.warmup, barrier)
        # keep the GPU under the same load while the sampler collects enough points
        t_end = time.perf_counter() + 0.6
        while time.perf_counter() < t_end:
            for _ in range(50):
                step()
            torch.cuda.synchronize()
    launches = args.steps
    assert tnn.launch_count() - n0 >= args.steps + args.warmup
    if tnn.device_status(local, True) != 0:
        raise RuntimeError("a bounded in-kernel wait gave up during the benchmark")

    t = torch.tensor([total], dtype=torch.float64, device=dev)
    if use_dist:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total = float(t.item())
    sec = total / args.steps
    value = w.flops * world / sec / 1e12

    # The timed region holds exactly one kernel, launched once per step, so its average launch
    # duration is the region's CUDA-event time over the steps (gaps between launches included).
    # Bracketing every launch with its own pair of events would also time the host's launch
    # preparation whenever the queue runs dry; that figure rides along as launch_ms_bracketed.
    launch_ms = sec * 1e3
    launch_ms_bracketed = per_launch_ms(step, max(args.steps, 20))
    achieved = w.flops / (launch_ms / 1e3) / 1e12
    traffic = NCU_TRAFFIC_BYTES.get(w.name)

    # end to end through the C ABI's host-buffer call: pinned host tensors in, host tensors out
    oh = torch.empty(qh.shape, dtype=torch.bfloat16).pin_memory()
    lseh = torch.empty(qh.shape[:3], dtype=torch.float32).pin_memory()
    for _ in range(2):
        tnn.sdpa_host(qh, kh, vh, is_causal=w.causal, out=oh, lse=lseh, device=local)
    barrier()
    t0 = time.perf_counter()
    e2e_steps = min(args.steps, 20)
    for _ in range(e2e_steps):
        tnn.sdpa_host(qh, kh, vh, is_causal=w.causal, out=oh, lse=lseh, device=local)
    e2e_sec = (time.perf_counter() - t0) / e2e_steps
    t = torch.tensor([e2e_sec], dtype=torch.float64, device=dev)
    if use_dist:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_sec = float(t.item())
    h2d = (qh.numel() + kh.numel() + vh.numel()) * 2
    d2h = oh.numel() * 2 + lseh.numel() * 4

    def all_max(x):
        tt = torch.tensor([x], dtype=torch.float64, device=dev)
        if use_dist:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item())

    sharded = None
    if use_dist and not args.no_others:
        sharded = sharded_workloads(tnn, dev, rank, world, barrier, all_max)

    line = None
    if rank == 0:
        cpu = None
        others = None
        if world == 1:
            torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
            flops, times = time_cpu(w, 3, 1)
            best = min(times)
            cpu = {"value": flops / best / 1e12, "unit": UNIT, "cores": torch.get_num_threads(),
                   "kind": "reference",
                   "sample": (f"full {w.name} batch, best of 3: ATen scaled_dot_product_attention (the call at "
                              f"cc/src/tyr.cpp:3941) on fp32 CPU tensors via torch {torch.__version__}, "
                              "repeat_interleave inside the timed call"),
                   "ms": best * 1e3, "host_cpus": os.cpu_count()}
            if not args.no_others:
                others = other_workloads(tnn, dev, peaks)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(w, world),
            "clocks": clocks.summary(),
            "e2e": {"value": w.flops * world / e2e_sec / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_sec * 1e3,
                    "api": "tyr_b200_attn_prefill_host (pinned host buffers)"},
            "gpu_launches": launches,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"],
                         "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"], "traffic": traffic,
                         "peak_source": peaks["source"] + " bf16_tflops (burst: kernel timed alone)",
                         "launch_ms": launch_ms, "launch_ms_bracketed": launch_ms_bracketed,
                         "frac_of_sustained": (achieved / peaks["bf16_tflops_sustained"]
                                               if peaks.get("bf16_tflops_sustained") else None),
                         "frac_of_nominal_2250": achieved / 2250.0},
            "cpu_baseline": cpu,
        }
        if others is not None:
            line["other_workloads"] = others
        if sharded is not None:
            line["strong_scaling_sharded"] = sharded
        print(json.dumps(line), flush=True)
    if use_dist:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=[n for n, w in W.WORKLOADS.items() if w.kind == "prefill"])
    ap.add_argument("--no-others", action="store_true", help="skip the extra kernel-only workloads")
    ap.add_argument("--profile", choices=["prefill", "backward", "decode"], default=None,
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
