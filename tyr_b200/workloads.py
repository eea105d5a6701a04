"""The five benchmark workloads as seeded synthetic inputs.

Model names denote shapes only: no weights, prompts or dataset items are used.
All draws come from one `torch.Generator(device="cpu")` per workload, in fp32, in
the order Q, K, V (decode: lengths, Q, then per sequence K, V) and are cast to
bf16 for the device.  A checker that wants fp32 inputs upcasts the bf16 values,
the reference's own fixture convention (Examples/GPU/RunFlashAttn.lean:30-36).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch


@dataclass(frozen=True)
class Workload:
    name: str
    kind: str          # "prefill" | "decode"
    batch: int
    n_head: int
    n_kv_head: int
    seq: int           # prefill: q_seq = kv_seq; decode: maximum KV length
    head_dim: int
    causal: bool
    seed: int
    qk_rmsnorm: bool   # Q, K RMS-normalised per head vector (QK-norm models)
    min_len: int = 0   # decode: lengths uniform in [min_len, seq]

    @property
    def flops(self) -> float:
        """4*B*Hq*Sq*Skv*D, halved for causal (prefill only)."""
        f = 4.0 * self.batch * self.n_head * self.seq * self.seq * self.head_dim
        return f / 2 if self.causal else f

    @property
    def io_bytes(self) -> int:
        """bf16 Q + K + V + O plus the fp32 LSE (prefill only)."""
        q = self.batch * self.n_head * self.seq * self.head_dim * 2
        kv = self.batch * self.n_kv_head * self.seq * self.head_dim * 2
        return 2 * q + 2 * kv + self.batch * self.n_head * self.seq * 4


WORKLOADS = {
    # the five benchmarked shapes (name, kind, batch, query heads, KV heads, sequence, head_dim, causal, seed, normalised Q/K)
    "gpt_char": Workload("gpt_char", "prefill", 64, 6, 6, 256, 64, True, 0, False),
    "qwen3_0p6b_prefill": Workload("qwen3_0p6b_prefill", "prefill", 8, 16, 8, 2048, 128, True, 1, True),
    "qwen3_8b_prefill": Workload("qwen3_8b_prefill", "prefill", 4, 32, 8, 8192, 128, True, 2, True),
    "qwen3_8b_decode": Workload("qwen3_8b_decode", "decode", 64, 32, 8, 32768, 128, False, 3, False, 512),
    "flux_mmdit": Workload("flux_mmdit", "prefill", 4, 24, 24, 4608, 128, False, 4, True),
}


def _rmsnorm(x: torch.Tensor) -> torch.Tensor:
    # nn.rmsNorm without weight: x / sqrt(mean(x^2) + eps)  (Tyr/Torch.lean:1122-1126)
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + 1e-6)


def _randn_chunked(shape, gen: torch.Generator) -> torch.Tensor:
    return torch.randn(shape, generator=gen, dtype=torch.float32)


def make_prefill(w: Workload, batch: Optional[int] = None, heads: Optional[Tuple[int, int]] = None,
                 seq: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """bf16 CPU tensors (q, k, v).  The optional overrides shrink the case for
    tests that need the CPU checker to finish in seconds."""
    assert w.kind == "prefill"
    B = batch or w.batch
    Hq, Hkv = heads or (w.n_head, w.n_kv_head)
    S = seq or w.seq
    gen = torch.Generator(device="cpu").manual_seed(w.seed)
    q = _randn_chunked((B, Hq, S, w.head_dim), gen)
    k = _randn_chunked((B, Hkv, S, w.head_dim), gen)
    v = _randn_chunked((B, Hkv, S, w.head_dim), gen)
    if w.qk_rmsnorm:
        q, k = _rmsnorm(q), _rmsnorm(k)
    return q.bfloat16(), k.bfloat16(), v.bfloat16()


def decode_lengths(w: Workload, batch: Optional[int] = None) -> List[int]:
    gen = torch.Generator(device="cpu").manual_seed(w.seed)
    return torch.randint(w.min_len, w.seq + 1, (batch or w.batch,), generator=gen).tolist()


def make_decode(w: Workload, batch: Optional[int] = None, max_len: Optional[int] = None,
                device: str = "cpu"):
    """(q [B,Hq,D] bf16, [K_b], [V_b], lengths).  K_b, V_b: [Hkv, L_b, D] bf16 contiguous.
    With `device` = a CUDA device the draws happen there per sequence (same seed
    stream is not preserved across devices; parity tests use device="cpu")."""
    assert w.kind == "decode"
    B = batch or w.batch
    gen = torch.Generator(device="cpu").manual_seed(w.seed)
    lens = torch.randint(w.min_len, w.seq + 1, (B,), generator=gen).tolist()
    if max_len is not None:
        lens = [1 + (L - 1) % max_len for L in lens]
    q = torch.randn((B, w.n_head, w.head_dim), generator=gen, dtype=torch.float32).bfloat16()
    ks, vs = [], []
    if device == "cpu":
        for L in lens:
            ks.append(torch.randn((w.n_kv_head, L, w.head_dim), generator=gen, dtype=torch.float32).bfloat16())
            vs.append(torch.randn((w.n_kv_head, L, w.head_dim), generator=gen, dtype=torch.float32).bfloat16())
    else:
        dgen = torch.Generator(device=device).manual_seed(w.seed)
        for L in lens:
            ks.append(torch.randn((w.n_kv_head, L, w.head_dim), generator=dgen, device=device,
                                  dtype=torch.float32).bfloat16())
            vs.append(torch.randn((w.n_kv_head, L, w.head_dim), generator=dgen, device=device,
                                  dtype=torch.float32).bfloat16())
    return q, ks, vs, lens


def decode_kv_bytes(lens: List[int], n_kv_head: int, head_dim: int) -> int:
    """Algorithmic bytes of one decode step: every K and V element once, bf16."""
    return sum(lens) * n_kv_head * head_dim * 2 * 2
