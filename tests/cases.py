"""Frozen test cases shared by the golden-vector generator and the tests.

The attention matrix and its seeds are those of the reference's GPU
differential suite (turboquant_kv/test_packed_attention_triton.py:51-68) and of
its frozen validation set (turboquant_kv/tsc/validation.py:192-207), followed by
cases this build adds (6-bit, mixed widths, 64-token pages, GQA 8).
Inputs are drawn in the reference's order: k, v, q from one seeded CPU
generator, which then also orders the pages.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class AttnCase:
    name: str
    seed: int
    B: int
    Hq: int
    Hkv: int
    D: int
    lens: tuple
    S: int
    bw_k: int
    bw_v: int
    q_scale: float = 1.0


ATTENTION_CASES = [
    AttnCase("qwen7b_gqa_short", 101, 3, 28, 4, 128, (1, 17, 64), 16, 8, 8),
    AttnCase("qwen7b_gqa_mixed", 102, 4, 28, 4, 128, (0, 300, 31, 129), 32, 8, 8),
    AttnCase("mha_like", 103, 2, 8, 8, 64, (40, 7), 16, 8, 8),
    AttnCase("gqa8_2", 104, 3, 8, 2, 64, (16, 33, 1), 16, 8, 8),
    AttnCase("huge_scores", 105, 2, 28, 4, 128, (90, 47), 16, 8, 8, 50.0),
    AttnCase("four_bit", 106, 2, 28, 4, 128, (77, 160), 16, 4, 4),
    AttnCase("three_bit", 107, 2, 8, 2, 128, (50, 19), 16, 3, 3),
    AttnCase("long_4k", 108, 2, 28, 4, 128, (4096, 2500), 32, 8, 8),
    AttnCase("batch32", 109, 32, 28, 4, 128, tuple(range(5, 5 + 32 * 61, 61)), 16, 8, 8),
    # frozen validation set, Llama-like family (32/8 heads, 4-bit, 16-token pages)
    AttnCase("val_edges", 1101, 4, 32, 8, 128, (0, 1, 16, 17), 16, 4, 4),
    AttnCase("val_tail", 1102, 3, 32, 8, 128, (47, 70, 5), 16, 4, 4),
    AttnCase("val_long", 1103, 2, 32, 8, 128, (1024, 517), 16, 4, 4),
    AttnCase("val_huge", 1104, 4, 32, 8, 128, (200, 33, 64, 9), 16, 4, 4, 40.0),
    # added here
    AttnCase("six_bit", 2001, 3, 32, 8, 128, (130, 16, 255), 16, 6, 6),
    AttnCase("mixed_4k_6v", 2002, 3, 32, 8, 128, (513, 40, 96), 16, 4, 6),
    AttnCase("page64_gqa8", 2003, 2, 64, 8, 128, (700, 64), 64, 4, 4),
    AttnCase("two_bit", 2004, 2, 8, 2, 128, (33, 80), 16, 2, 2),
    AttnCase("five_bit", 2005, 2, 8, 4, 64, (20, 65), 16, 5, 5),
    AttnCase("tiny_dim", 2006, 2, 4, 2, 16, (9, 30), 8, 8, 8),
    AttnCase("mqa_gqa7", 2007, 2, 7, 1, 128, (100, 3), 16, 4, 4),
]


def attention_inputs(c: AttnCase):
    """Dense k, v (B, Hkv, Lmax, D), q (B, Hq, 1, D) and the generator, in the
    state the page assignment expects."""
    g = torch.Generator().manual_seed(c.seed)
    Lmax = max(max(c.lens), 1)
    k = torch.randn(c.B, c.Hkv, Lmax, c.D, generator=g)
    v = torch.randn(c.B, c.Hkv, Lmax, c.D, generator=g)
    q = torch.randn(c.B, c.Hq, 1, c.D, generator=g) * c.q_scale
    return k, v, q, g


@dataclass(frozen=True)
class QuantCase:
    name: str
    seed: int
    shape: tuple            # leading shape; vectors = prod(shape)
    D: int
    bw: int
    dtype: str = "float32"
    kind: str = "normal"    # normal | outlier | zero_rows | tiny | huge


QUANT_CASES = [
    QuantCase("one_vector", 11, (1,), 128, 4),
    QuantCase("two_vectors", 12, (2,), 128, 4),
    QuantCase("five_vectors", 13, (5,), 128, 6),
    QuantCase("six_vectors", 14, (6,), 128, 4),
    QuantCase("decode_2x8", 15, (2, 8, 1), 128, 4, "float16", "outlier"),
    QuantCase("decode_6bit", 16, (4, 8, 1), 128, 6, "float16", "outlier"),
    QuantCase("prefill_bf16", 17, (1, 4, 33), 128, 4, "bfloat16", "outlier"),
    QuantCase("eight_bit", 18, (3, 2, 7), 128, 8),
    QuantCase("three_bit", 19, (2, 2, 9), 128, 3),
    QuantCase("two_bit", 20, (2, 3, 5), 128, 2),
    QuantCase("five_bit", 21, (2, 3, 5), 128, 5),
    QuantCase("dim64", 22, (2, 4, 11), 64, 4),
    QuantCase("dim64_small", 23, (3,), 64, 6),
    QuantCase("dim16", 24, (3, 2, 7), 16, 8),
    QuantCase("dim8", 25, (4, 5), 8, 4),
    QuantCase("zero_rows", 26, (2, 2, 6), 128, 4, "float32", "zero_rows"),
    QuantCase("zero_rows_6bit", 27, (2, 2, 6), 128, 6, "float32", "zero_rows"),
    QuantCase("tiny_values", 28, (12,), 128, 4, "float32", "tiny"),
    QuantCase("huge_values", 29, (12,), 128, 4, "float32", "huge"),
    QuantCase("many", 30, (16, 8, 16), 128, 4, "float16", "outlier"),
]


def quant_input(c: QuantCase) -> torch.Tensor:
    g = torch.Generator().manual_seed(c.seed)
    x = torch.randn(*c.shape, c.D, generator=g)
    if c.kind == "outlier":
        x[..., :3] *= 8.0
    elif c.kind == "zero_rows":
        flat = x.view(-1, c.D)
        flat[1] = 0.0
        flat[-1] = 0.0
    elif c.kind == "tiny":
        x *= 1e-30
    elif c.kind == "huge":
        x *= 1e4
    return x.to(getattr(torch, c.dtype))


@dataclass(frozen=True)
class AppendCase:
    name: str
    seed: int
    B: int
    Hkv: int
    D: int
    S: int
    bw_k: int
    bw_v: int
    lengths: tuple      # tokens already stored per sequence
    n: int              # tokens appended per sequence
    layers: int = 2
    dtype: str = "float32"


APPEND_CASES = [
    AppendCase("decode_b3", 31, 3, 2, 128, 16, 4, 4, (0, 15, 16), 1),
    AppendCase("decode_rows2", 32, 1, 2, 128, 16, 4, 4, (37,), 1),
    AppendCase("decode_rows4_f16", 33, 2, 2, 128, 16, 6, 6, (5, 31), 1, 2, "float16"),
    AppendCase("prefill_chunk", 34, 1, 4, 128, 16, 4, 4, (10,), 23, 2, "bfloat16"),
    AppendCase("batch_prefill", 35, 2, 2, 64, 8, 8, 8, (3, 8), 9),
    AppendCase("mixed_widths", 36, 4, 8, 128, 16, 4, 6, (100, 0, 47, 16), 1, 1, "float16"),
]


def append_input(c: AppendCase, layer: int):
    g = torch.Generator().manual_seed(c.seed * 100 + layer)
    k = torch.randn(c.B, c.Hkv, c.n, c.D, generator=g)
    v = torch.randn(c.B, c.Hkv, c.n, c.D, generator=g)
    k[..., :2] *= 8.0
    dt = getattr(torch, c.dtype)
    return k.to(dt), v.to(dt)


def append_pool_pages(c: AppendCase) -> int:
    return sum(-(-(L + c.n) // c.S) for L in c.lengths) + 2
