"""Seeded synthetic Q/K/V for the five benchmark configurations.

The reference ships no data (its tests load absent .pt files), so every workload here is generated
from a seed.  Heads are generated independently from `seed + global_head_id`, so a rank that owns
heads [h0, h1) of a (batch x head) split reproduces exactly the slices of the single-GPU tensor.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch


@dataclass(frozen=True)
class Workload:
    name: str
    B: int
    H: int
    S: int
    D: int
    kind: str            # "normal" | "clustered"
    sigma: float = 1.0   # std of the i.i.d. normal inputs ("normal") / of v ("clustered")
    centroids: int = 0
    run: int = 0
    centroid_std: float = 2.0
    noise_std: float = 0.5
    tau: float = 1e-3
    dtype: str = "bf16"
    seed: int = 0


WORKLOADS = {
    # CPU-runnable reference case
    "c1": Workload("c1_cpu_b1h4s1024d64", 1, 4, 1024, 64, "normal", tau=1e-3, dtype="fp32", seed=1000),
    # dense full attention
    "c2": Workload("c2_dense_b2h16s4096d64", 2, 16, 4096, 64, "normal", sigma=0.5, tau=1e-3, seed=2000),
    # clustered threshold sparse attention: the headline configuration
    "c3": Workload("c3_clustered_b1h32s16384d128", 1, 32, 16384, 128, "clustered", centroids=64, run=256,
                   tau=1e-4, seed=3000),
    # ragged sequence length
    "c4": Workload("c4_ragged_b4h24s12345d64", 4, 24, 12345, 64, "clustered", centroids=64, run=128,
                   tau=1e-3, seed=4000),
    # long context, sharded over (batch x head)
    "c5": Workload("c5_long_b8h64s65536d128", 8, 64, 65536, 128, "clustered", centroids=256, run=512,
                   tau=1e-4, seed=5000),
}


def _gen(device, seed: int) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def make_head(w: Workload, head_id: int, device="cpu") -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """fp32 (q, k, v), each [S, D], for global head `head_id` in [0, B*H)."""
    g = _gen(device, w.seed + head_id)
    S, D = w.S, w.D
    if w.kind == "normal":
        q = torch.randn(S, D, generator=g, device=device) * w.sigma
        k = torch.randn(S, D, generator=g, device=device) * w.sigma
        v = torch.randn(S, D, generator=g, device=device) * w.sigma
        return q, k, v
    cent = torch.randn(w.centroids, D, generator=g, device=device) * w.centroid_std
    n_runs = (S + w.run - 1) // w.run
    out = []
    for _ in range(2):                                   # q then k: independent run->centroid draws
        pick = torch.randint(0, w.centroids, (n_runs,), generator=g, device=device)
        base = cent[pick].repeat_interleave(w.run, dim=0)[:S]
        out.append(base + torch.randn(S, D, generator=g, device=device) * w.noise_std)
    v = torch.randn(S, D, generator=g, device=device) * w.sigma
    return out[0], out[1], v


def make_qkv(w: Workload, device="cpu", heads: Optional[range] = None, dtype: Optional[torch.dtype] = None):
    """(q, k, v) [1, n_heads, S, D] for the global heads in `heads` (default: all B*H, returned as
    [B, H, S, D]).  dtype defaults to bf16 for the bf16 workloads and fp32 for c1."""
    if dtype is None:
        dtype = torch.float32 if w.dtype == "fp32" else torch.bfloat16
    all_heads = heads is None
    heads = range(w.B * w.H) if all_heads else heads
    n = len(heads)
    q = torch.empty(n, w.S, w.D, dtype=dtype, device=device)
    k = torch.empty_like(q)
    v = torch.empty_like(q)
    for i, hid in enumerate(heads):
        qh, kh, vh = make_head(w, hid, device)
        q[i], k[i], v[i] = qh.to(dtype), kh.to(dtype), vh.to(dtype)
    shape = (w.B, w.H, w.S, w.D) if all_heads else (1, n, w.S, w.D)
    return q.view(shape), k.view(shape), v.view(shape)


def shard_heads(total_heads: int, world_size: int, rank: int) -> range:
    """Contiguous split of the flattened (batch x head) units over ranks; the first
    `total_heads % world_size` ranks take one extra unit."""
    base, extra = divmod(total_heads, world_size)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))
