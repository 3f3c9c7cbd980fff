"""Seeded synthetic workloads in the shapes the decode path is measured and tested on.

The reference measures on key/query vectors dumped from Llama-3-8B layers
(benchmark_area/kv_sampling/collect_kv_data.py:321-422); those dumps are not distributed
with it, so the five configurations below take its shapes (D = 128, per-head key sets, unit
queries, top-k / percentile thresholds) with stated synthetic distributions instead:

  cfg0  fp32, 1 x 8 heads x 4,096 keys, N(0,1) scaled per channel by exp(N(0, 0.5)); one
        query per head; 2 levels, branching 64; tau = 128th largest q.k per head
  cfg1  bf16, 32 query / 8 KV heads, batch 1, context 32,768; N(0,1) with RoPE (base 500000)
        by position on the keys and 4 outlier channels x8; 3 levels, branching 32; tau keeps 2 %
  cfg2  cfg1 with batch 16 and context 131,072 (the headline decode step)
  cfg3  streaming update: prefix 65,536 keys (cfg1 distribution), 8 KV heads, 4,096 single-key
        appends, full rebuild every 1,024
  cfg4  64 query / 8 KV heads, bf16, sequence shards of 131,072 keys (cfg1 distribution) per
        GPU, 3 levels, branching 64

Both bench.py and the parity tests draw their inputs from here, so the kernels are tested
on the data they are timed on.  Everything is generated per head from a torch.Generator,
so a prefix of the heads / tokens of a configuration is reproducible on its own.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

DIM = 128
ROPE_BASE = 500000.0
OUTLIER_CHANNELS = (7, 42, 71, 110)
OUTLIER_SCALE = 8.0


@dataclass(frozen=True)
class Workload:
    name: str
    batch: int
    kv_heads: int
    q_heads: int
    context: int
    levels: int
    branching: int
    dtype: torch.dtype
    dist: str                 # "rope_outlier" | "aniso" | "clustered"
    keep: float               # fraction of keys tau keeps (exact k-th largest score per query head)
    seed: int = 0

    @property
    def group(self) -> int:
        return self.q_heads // self.kv_heads

    @property
    def kth(self) -> int:
        return max(1, int(round(self.keep * self.context)))


CFG0 = Workload("cfg0_cpu_ctx4096", 1, 8, 8, 4096, 2, 64, torch.float32, "aniso", 128 / 4096)
CFG1 = Workload("cfg1_b1_ctx32768", 1, 8, 32, 32768, 3, 32, torch.bfloat16, "rope_outlier", 0.02)
CFG2 = Workload("cfg2_b16_ctx131072", 16, 8, 32, 131072, 3, 32, torch.bfloat16, "rope_outlier", 0.02)
CFG3 = Workload("cfg3_streaming_prefix65536", 1, 8, 32, 65536, 3, 32, torch.bfloat16, "rope_outlier", 0.02)
CFG4 = Workload("cfg4_seqshard_131072_per_gpu", 1, 8, 64, 131072, 3, 64, torch.bfloat16, "rope_outlier", 0.02)
# control: cfg1's shape on clustered keys (not a BASELINE configuration)
CLUSTERED = Workload("clustered_b1_ctx32768", 1, 8, 32, 32768, 3, 32, torch.bfloat16, "clustered", 0.02)
CONFIGS = {w.name.split("_")[0]: w for w in (CFG0, CFG1, CFG2, CFG3, CFG4)}


def rope_(x: torch.Tensor, positions: torch.Tensor, base: float = ROPE_BASE) -> torch.Tensor:
    """Llama half-rotation RoPE, in place on (..., L, D) with positions (L,)."""
    d = x.shape[-1]
    inv = 1.0 / (base ** (torch.arange(0, d, 2, device=x.device, dtype=torch.float32) / d))
    ang = positions.to(torch.float32)[:, None] * inv[None, :]
    cos, sin = ang.cos(), ang.sin()
    x1, x2 = x[..., : d // 2].float(), x[..., d // 2:].float()
    r1 = x1 * cos - x2 * sin
    r2 = x2 * cos + x1 * sin
    x[..., : d // 2] = r1.to(x.dtype)
    x[..., d // 2:] = r2.to(x.dtype)
    return x


def aniso_scale(seed: int, device, dim: int = DIM) -> torch.Tensor:
    """Per-channel scale exp(N(0, 0.5)) of the "aniso" distribution, drawn once per seed."""
    g = torch.Generator(device=device)
    g.manual_seed(seed * 7919 + 11)
    return torch.exp(torch.randn((dim,), generator=g, device=device) * 0.5)


def make_kv(n_heads: int, n: int, seed: int, device, *, dist: str = "rope_outlier", dtype=torch.bfloat16,
            first_pos: int = 0, dim: int = DIM) -> Tuple[torch.Tensor, torch.Tensor]:
    """keys, values (n_heads, n, dim) in `dtype` on `device`, generated head by head.
    Head i of seed s equals head 0 of a one-head call only when generated in the same
    sequence; the tests and the bench both start from head 0."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    keys = torch.empty((n_heads, n, dim), dtype=dtype, device=device)
    vals = torch.empty((n_heads, n, dim), dtype=dtype, device=device)
    pos = torch.arange(first_pos, first_pos + n, device=device)
    scale = aniso_scale(seed, device, dim) if dist == "aniso" else None
    for i in range(n_heads):
        k = torch.randn((n, dim), generator=g, device=device, dtype=torch.float32)
        if dist == "rope_outlier":
            rope_(k, pos)
            k[:, list(OUTLIER_CHANNELS)] *= OUTLIER_SCALE
        elif dist == "aniso":
            k *= scale
        elif dist == "clustered":
            # a mixture of 1,024 tight clusters (centres N(0, 9 I), spread 0.05): data on which ball
            # pruning has something to prune -- not one of the reference's distributions, a control
            cent = torch.randn((1024, dim), generator=g, device=device, dtype=torch.float32) * 3.0
            which = torch.randint(0, 1024, (n,), generator=g, device=device)
            k = cent[which] + 0.05 * k
        else:
            raise ValueError(f"unknown distribution {dist!r}")
        keys[i] = k.to(dtype)
        vals[i] = torch.randn((n, dim), generator=g, device=device, dtype=torch.float32).to(dtype)
    return keys, vals


def make_queries(n_qheads: int, seed: int, device, *, pos: Optional[int] = None, dim: int = DIM) -> torch.Tensor:
    """(n_qheads, dim) fp32 N(0,1) queries; RoPE at position `pos` when given."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    q = torch.randn((n_qheads, 1, dim), generator=g, device=device, dtype=torch.float32)
    if pos is not None:
        rope_(q, torch.tensor([pos], device=device))
    return q[:, 0, :].contiguous()


def make_inputs(w: Workload, device, *, n_heads: Optional[int] = None, context: Optional[int] = None,
                seed_offset: int = 0):
    """keys, values for the first `n_heads` (batch, kv head) groups of `w` (default: all) over
    `context` tokens (default: all), and one fp32 query per query head of those groups."""
    h = w.batch * w.kv_heads if n_heads is None else n_heads
    n = w.context if context is None else context
    keys, vals = make_kv(h, n, 1000 + w.seed + seed_offset, device, dist=w.dist, dtype=w.dtype)
    q = make_queries(h * w.group, 50 + w.seed + seed_offset, device,
                     pos=n if w.dist == "rope_outlier" else None)
    return keys, vals, q


def random_centres(n_heads: int, n: int, k: int, seed: int, device) -> torch.Tensor:
    """k distinct positions in [0, n) per head (initial centres: random data points,
    as CUDAIndexer picks them, indexer/cuda.py:229-237)."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return torch.rand((n_heads, n), generator=g, device=device).topk(k, dim=1).indices.to(torch.int32).contiguous()


def guard_banded_tau(scores: torch.Tensor, kth: int) -> torch.Tensor:
    """Midpoint between the kth and (kth+1)th largest score of each row: a threshold no key
    sits on, as the reference's exact-set tests choose it (tests/test_customized.py:77-83)."""
    n = scores.shape[-1]
    srt = torch.sort(scores, dim=-1, descending=True).values
    kth = min(max(1, kth), n - 1)
    return (0.5 * (srt[:, kth - 1].double() + srt[:, kth].double())).float().contiguous()
