"""Seeded synthetic inputs for the five benchmark configurations.

The reference names no dataset for this path; these tensors are the workload.
Everything is drawn on the CPU from one `torch.Generator` so that the CUDA
path, the CPU oracle and the committed golden vectors see identical inputs.

Distribution (all configs): K, V ~ N(0, 1); `round(0.02 * D)` channels (the
first ones of a seeded `randperm(D)`, the same for K and V) are scaled by 8 as
outliers; q ~ N(0, 1) / sqrt(D).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch


@dataclass(frozen=True)
class Workload:
    name: str
    batch: int
    q_heads: int
    kv_heads: int
    head_dim: int
    page_size: int
    bits_k: int
    bits_v: int
    dtype: torch.dtype
    context: int | None = None          # uniform context, or None for ragged
    ragged: tuple[int, int] | None = None   # (lo, hi) log-uniform bounds
    seed: int = 0

    def seq_lens(self) -> list[int]:
        if self.context is not None:
            return [self.context] * self.batch
        lo, hi = self.ragged
        g = torch.Generator().manual_seed(self.seed + 7919)
        u = torch.rand(self.batch, generator=g, dtype=torch.float64)
        return [int(round(math.exp(math.log(lo) + float(x) * (math.log(hi) - math.log(lo)))))
                for x in u]

    def bytes_per_token_head(self) -> int:
        return self.head_dim * self.bits_k // 8 + self.head_dim * self.bits_v // 8 + 4

    def algorithmic_bytes(self, kv_heads: int | None = None, q_heads: int | None = None) -> int:
        """Bytes one decode step must move: codes + fp16 norms of every cached
        token, the used page-table entries, q in and out."""
        hkv = self.kv_heads if kv_heads is None else kv_heads
        hq = self.q_heads if q_heads is None else q_heads
        lens = self.seq_lens()
        el = torch.empty((), dtype=self.dtype).element_size()
        pages = sum(-(-L // self.page_size) for L in lens)
        return (sum(lens) * hkv * self.bytes_per_token_head() + 4 * pages
                + self.batch * hq * self.head_dim * 2 * el)


WORKLOADS = {
    "config1": Workload("config1", 1, 8, 2, 128, 16, 4, 4, torch.float32, context=1024),
    "config2": Workload("config2", 16, 32, 8, 128, 16, 4, 4, torch.float16, context=8192),
    "config3": Workload("config3", 32, 32, 8, 128, 16, 6, 6, torch.float16, context=16384),
    "config4": Workload("config4", 1, 64, 8, 128, 64, 4, 4, torch.float16, context=131072),
    "config5": Workload("config5", 128, 32, 8, 128, 16, 4, 6, torch.float16, ragged=(512, 32768)),
    "headline32k": Workload("headline32k", 16, 32, 8, 128, 16, 4, 4, torch.float16, context=32768),
}


def outlier_channels(head_dim: int, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed + 104729)
    return torch.randperm(head_dim, generator=g)[: int(round(0.02 * head_dim))]


def dense_kv(w: Workload, seq: int, kv_head_slice: slice | None = None):
    """Dense K, V of one sequence: (Hkv, L, D) each, in the workload dtype.

    Sequences are drawn independently (one generator per sequence) so a rank
    that owns a subset of kv heads or a test that needs one sequence can build
    just that part and still agree with a full build.
    """
    L = w.seq_lens()[seq]
    g = torch.Generator().manual_seed(w.seed * 1000003 + seq)
    k = torch.randn(w.kv_heads, L, w.head_dim, generator=g)
    v = torch.randn(w.kv_heads, L, w.head_dim, generator=g)
    ch = outlier_channels(w.head_dim, w.seed)
    k[..., ch] *= 8.0
    v[..., ch] *= 8.0
    k, v = k.to(w.dtype), v.to(w.dtype)
    if kv_head_slice is not None:
        k, v = k[kv_head_slice], v[kv_head_slice]
    return k, v


def queries(w: Workload) -> torch.Tensor:
    """(B, Hq, 1, D) decode queries in the workload dtype."""
    g = torch.Generator().manual_seed(w.seed * 1000003 + 999983)
    q = torch.randn(w.batch, w.q_heads, 1, w.head_dim, generator=g) / math.sqrt(w.head_dim)
    return q.to(w.dtype)


def new_tokens(w: Workload, step: int = 0):
    """K, V of one appended token per sequence: (B, Hkv, 1, D)."""
    g = torch.Generator().manual_seed(w.seed * 1000003 + 500009 + step)
    k = torch.randn(w.batch, w.kv_heads, 1, w.head_dim, generator=g)
    v = torch.randn(w.batch, w.kv_heads, 1, w.head_dim, generator=g)
    ch = outlier_channels(w.head_dim, w.seed)
    k[..., ch] *= 8.0
    v[..., ch] *= 8.0
    return k.to(w.dtype), v.to(w.dtype)


def page_assignment(w: Workload, spare_pages: int = 0):
    """Random page table over a contiguous pool: (table (B, max_pages) int32
    with -1 padding, number of pages in the pool)."""
    lens = w.seq_lens()
    need = [-(-L // w.page_size) for L in lens]
    total = sum(need) + spare_pages
    g = torch.Generator().manual_seed(w.seed * 1000003 + 15485863)
    order = torch.randperm(total, generator=g).to(torch.int32)
    table = torch.full((w.batch, max(max(need), 1)), -1, dtype=torch.int32)
    at = 0
    for b, n in enumerate(need):
        table[b, :n] = order[at:at + n]
        at += n
    return table, total
