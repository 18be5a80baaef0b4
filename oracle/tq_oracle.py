"""TEST INFRASTRUCTURE ONLY: CPU oracle for the TurboQuant packed-KV path.

This module restates, on the CPU, what lgoyal6/winnow's ``turboquant_kv``
computes on the path the CUDA kernels replace.  Only ``tests/``, the smoke
check and the benchmark's CPU-baseline leg may import it; the product package
never does, and it raises if its CUDA library is missing rather than falling
back to anything in here.

Parity status: PINNED.  ``tests/golden/`` holds vectors produced by importing
the reference itself (script committed beside them); ``tests/test_oracle.py``
checks every function below against them bit for bit (bytes, indices, norms,
codebooks) or to 2e-4 (attention outputs, the reference's own CPU tolerance).

Reference map (file:line in the reference project):
  packed_bytes / pack / unpack      turboquant_kv/packing.py:24-89
  lloyd_max_gaussian                turboquant_kv/cache.py:62-82
  OracleQuantizer                   turboquant_kv/cache.py:85-115
  pages_from_dense                  turboquant_kv/packed_attention.py:341-377
  check_layout                      turboquant_kv/packed_attention.py:114-163
  reconstruct_attention             turboquant_kv/packed_attention.py:212-235
  tiled_attention / merge_states    turboquant_kv/packed_attention.py:260-334
  append_tokens                     turboquant_kv/packed_backend.py:135-170
  dequantize_rows                   turboquant_kv/cache.py:117-131

Byte and integer work and the order-sensitive fp32 arithmetic of ``quantize``
run in plain C (``tq_oracle.c``, which documents the summation orders); the
attention operators are fp32 torch on the CPU.
"""
from __future__ import annotations

import ctypes
import math
import os
import subprocess
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "_build" / "libtq_oracle.so"
_lib = None

SUPPORTED_WIDTHS = (2, 3, 4, 5, 6, 8)
ORDER_SEQUENTIAL = 0
ORDER_INTERLEAVED16 = 1


def build_c_oracle(force: bool = False) -> Path:
    """Compile tq_oracle.c with the Makefile beside it (gcc only)."""
    src = _HERE / "tq_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B" if force else "-s", "all"],
                       check=True, capture_output=True)
    return _LIB_PATH


def _c():
    global _lib
    if _lib is None:
        build_c_oracle()
        lib = ctypes.CDLL(str(_LIB_PATH))
        vp, i64, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
        lib.tq_quantize.argtypes = [vp, i64, i32, vp, vp, i32, i32, vp, vp]
        lib.tq_pack.argtypes = [vp, i64, i32, i32, vp]
        lib.tq_unpack.argtypes = [vp, i64, i32, i32, vp]
        lib.tq_dequantize.argtypes = [vp, vp, i64, i32, vp, vp, vp]
        lib.tq_rotation_order_for_rows.argtypes = [i64]
        lib.tq_rotation_order_for_rows.restype = i32
        for f in (lib.tq_quantize, lib.tq_pack, lib.tq_unpack, lib.tq_dequantize):
            f.restype = None
        _lib = lib
    return _lib


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


# --------------------------------------------------------------------------
# layout
# --------------------------------------------------------------------------
def packed_bytes(head_dim: int, bit_width: int) -> int:
    bits = head_dim * bit_width
    if bits % 8:
        raise ValueError(f"head_dim*bit_width must be a multiple of 8, got "
                         f"{head_dim}*{bit_width}={bits}")
    return bits // 8


def pack(idx: torch.Tensor, bit_width: int) -> torch.Tensor:
    """(..., D) uint8 -> (..., D*bw/8) uint8, LSB-first bit stream."""
    D = idx.shape[-1]
    nb = packed_bytes(D, bit_width)
    src = np.ascontiguousarray(idx.detach().cpu().numpy().astype(np.uint8)).reshape(-1, D)
    out = np.empty((src.shape[0], nb), dtype=np.uint8)
    _c().tq_pack(_ptr(src), src.shape[0], D, bit_width, _ptr(out))
    return torch.from_numpy(out).reshape(*idx.shape[:-1], nb)


def unpack(packed: torch.Tensor, bit_width: int, head_dim: int) -> torch.Tensor:
    nb = packed.shape[-1]
    if nb != packed_bytes(head_dim, bit_width):
        raise ValueError("row length does not match head_dim*bit_width/8")
    src = np.ascontiguousarray(packed.detach().cpu().numpy()).reshape(-1, nb)
    out = np.empty((src.shape[0], head_dim), dtype=np.uint8)
    _c().tq_unpack(_ptr(src), src.shape[0], head_dim, bit_width, _ptr(out))
    return torch.from_numpy(out).reshape(*packed.shape[:-1], head_dim)


# --------------------------------------------------------------------------
# quantizer
# --------------------------------------------------------------------------
def lloyd_max_gaussian(levels: int, sigma: float = 1.0, iters: int = 200, tol: float = 1e-12):
    """Lloyd-Max centroids and bucket edges for N(0, sigma^2), float64.

    Start from `levels` points evenly spaced on [-3 sigma, 3 sigma]; each round
    puts the edges midway between neighbours and moves every centroid to the
    conditional mean of its bucket; stop when no centroid moves more than tol.
    """
    from scipy.stats import norm

    c = np.linspace(-3.0 * sigma, 3.0 * sigma, levels)
    for _ in range(iters):
        edges = np.concatenate(([-np.inf], 0.5 * (c[:-1] + c[1:]), [np.inf]))
        z = edges / sigma
        mass = norm.cdf(z[1:]) - norm.cdf(z[:-1])
        mean = sigma * (norm.pdf(z[:-1]) - norm.pdf(z[1:]))
        with np.errstate(divide="ignore", invalid="ignore"):
            moved = np.where(mass < 1e-300, c, mean / mass)
        done = np.max(np.abs(moved - c)) < tol
        c = moved
        if done:
            break
    edges = np.concatenate(([-np.inf], 0.5 * (c[:-1] + c[1:]), [np.inf]))
    return c, edges


def rotation_matrix(head_dim: int, seed: int) -> torch.Tensor:
    """Pi = Q * sign(diag R) of the QR of a CPU-seeded Gaussian matrix."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    G = torch.randn(head_dim, head_dim, generator=gen, dtype=torch.float32)
    Q, R = torch.linalg.qr(G)
    s = torch.sign(torch.diag(R))
    s[s == 0] = 1.0
    return (Q * s.unsqueeze(0)).contiguous()


_QUANTIZERS: dict = {}


class OracleQuantizer:
    def __init__(self, bit_width: int, head_dim: int, rotation_seed: int = 42):
        self.bit_width, self.head_dim = bit_width, head_dim
        self.Pi = rotation_matrix(head_dim, rotation_seed)
        c, edges = lloyd_max_gaussian(2 ** bit_width, sigma=1.0 / math.sqrt(head_dim))
        self.centroids = torch.tensor(c, dtype=torch.float32)
        self.boundaries = torch.tensor(edges[1:-1], dtype=torch.float32)

    @classmethod
    def get(cls, bit_width, head_dim, seed=42) -> "OracleQuantizer":
        key = (bit_width, head_dim, seed)
        if key not in _QUANTIZERS:
            _QUANTIZERS[key] = cls(bit_width, head_dim, seed)
        return _QUANTIZERS[key]

    def quantize(self, x: torch.Tensor, order: int | None = None):
        """(..., D) -> uint8 indices (..., D), fp32 norms (...,).

        `order=None` picks the rotation's summation order from the number of
        vectors in this call, as the reference's BLAS does (see tq_oracle.c).
        """
        D = self.head_dim
        flat = np.ascontiguousarray(x.detach().cpu().float().numpy()).reshape(-1, D)
        rows = flat.shape[0]
        if order is None:
            order = _c().tq_rotation_order_for_rows(rows)
        idx = np.empty((rows, D), dtype=np.uint8)
        norms = np.empty((rows,), dtype=np.float32)
        Pi = np.ascontiguousarray(self.Pi.numpy())
        b = np.ascontiguousarray(self.boundaries.numpy())
        _c().tq_quantize(_ptr(flat), rows, D, _ptr(Pi), _ptr(b), b.shape[0], order,
                         _ptr(idx), _ptr(norms))
        return (torch.from_numpy(idx).reshape(x.shape),
                torch.from_numpy(norms).reshape(x.shape[:-1]))


def dequantize_rows(packed: torch.Tensor, norms: torch.Tensor, centroids: torch.Tensor,
                    Pi: torch.Tensor, bit_width: int, head_dim: int) -> torch.Tensor:
    """(..., NB) packed rows + (...,) norms -> (..., D) fp32 reconstruction."""
    idx = np.ascontiguousarray(unpack(packed, bit_width, head_dim).numpy()).reshape(-1, head_dim)
    n = np.ascontiguousarray(norms.detach().cpu().float().numpy()).reshape(-1)
    out = np.empty((idx.shape[0], head_dim), dtype=np.float32)
    _c().tq_dequantize(_ptr(idx), _ptr(n), idx.shape[0], head_dim,
                       _ptr(np.ascontiguousarray(Pi.numpy())),
                       _ptr(np.ascontiguousarray(centroids.numpy())), _ptr(out))
    return torch.from_numpy(out).reshape(*packed.shape[:-1], head_dim)


# --------------------------------------------------------------------------
# paged cache model
# --------------------------------------------------------------------------
@dataclass
class OracleKV:
    k_pages: torch.Tensor      # (P, Hkv, S, NBk) uint8
    k_norms: torch.Tensor      # (P, Hkv, S) fp16
    v_pages: torch.Tensor
    v_norms: torch.Tensor
    page_table: torch.Tensor   # (B, max_pages) int32, -1 padded
    seq_lens: torch.Tensor     # (B,) int32
    k_Pi: torch.Tensor
    k_centroids: torch.Tensor
    k_bits: int
    v_Pi: torch.Tensor
    v_centroids: torch.Tensor
    v_bits: int
    head_dim: int

    @property
    def page_size(self):
        return self.k_pages.shape[2]

    @property
    def num_kv_heads(self):
        return self.k_pages.shape[1]


def pages_from_dense(k, v, seq_lens, k_tq: OracleQuantizer, v_tq: OracleQuantizer,
                     page_size: int, num_pages: int | None = None,
                     generator: torch.Generator | None = None) -> OracleKV:
    """Quantize dense (B, Hkv, Lmax, D) K/V into randomly ordered pages.

    Follows the reference fixture builder: page ids come from one
    `torch.randperm(total, generator)` consumed in (sequence, page) order, and
    each (sequence, page) slab of Hkv x tokens vectors is quantized in its own
    call, which fixes the rotation's summation order for short tails.
    """
    B, Hkv, _, D = k.shape
    lens = [int(x) for x in seq_lens]
    need = [-(-L // page_size) for L in lens]
    total = num_pages or max(sum(need), 1)
    order = torch.randperm(total, generator=generator).tolist()
    nbk, nbv = packed_bytes(D, k_tq.bit_width), packed_bytes(D, v_tq.bit_width)
    kp = torch.zeros(total, Hkv, page_size, nbk, dtype=torch.uint8)
    vp = torch.zeros(total, Hkv, page_size, nbv, dtype=torch.uint8)
    kn = torch.zeros(total, Hkv, page_size, dtype=torch.float16)
    vn = torch.zeros(total, Hkv, page_size, dtype=torch.float16)
    table = torch.full((B, max(max(need), 1)), -1, dtype=torch.int32)
    cursor = 0
    for b in range(B):
        for t in range(need[b]):
            pid = order[cursor]
            cursor += 1
            table[b, t] = pid
            lo, hi = t * page_size, min((t + 1) * page_size, lens[b])
            for dense, tq, pages, norms in ((k, k_tq, kp, kn), (v, v_tq, vp, vn)):
                idx, nrm = tq.quantize(dense[b, :, lo:hi])
                pages[pid, :, :hi - lo] = pack(idx, tq.bit_width)
                norms[pid, :, :hi - lo] = nrm.to(torch.float16)
    return OracleKV(kp, kn, vp, vn, table, torch.tensor(lens, dtype=torch.int32),
                    k_tq.Pi, k_tq.centroids, k_tq.bit_width,
                    v_tq.Pi, v_tq.centroids, v_tq.bit_width, D)


def append_tokens(kv_k_pages, kv_k_norms, kv_v_pages, kv_v_norms, page_table, lengths,
                  k, v, k_tq: OracleQuantizer, v_tq: OracleQuantizer) -> None:
    """Write n new tokens per sequence into one layer's pages, in place.

    k, v are (B, Hkv, n, D); sequence b's token i lands at position
    lengths[b] + i, i.e. page `page_table[b, pos // S]`, slot `pos % S`.  The
    whole (B, Hkv, n) slab is quantized in one call, as the reference does.
    """
    B, Hkv, n, D = k.shape
    S = kv_k_pages.shape[2]
    for dense, tq, pages, norms in ((k, k_tq, kv_k_pages, kv_k_norms),
                                    (v, v_tq, kv_v_pages, kv_v_norms)):
        idx, nrm = tq.quantize(dense)
        rows = pack(idx, tq.bit_width)
        for b in range(B):
            for i in range(n):
                pos = int(lengths[b]) + i
                pid = int(page_table[b, pos // S])
                pages[pid, :, pos % S] = rows[b, :, i]
                norms[pid, :, pos % S] = nrm[b, :, i].to(torch.float16)


class LayoutError(ValueError):
    pass


def check_layout(q: torch.Tensor, kv: OracleKV) -> None:
    if q.dim() != 4:
        raise LayoutError("q must be (B, Hq, Q, D)")
    B, Hq, _, D = q.shape
    P, Hkv, S = kv.k_pages.shape[:3]
    if D != kv.head_dim or Hq % Hkv:
        raise LayoutError("head_dim or head-count mismatch")
    if kv.page_table.dtype != torch.int32 or kv.seq_lens.dtype != torch.int32:
        raise LayoutError("page_table and seq_lens must be int32")
    if kv.page_table.dim() != 2 or kv.page_table.shape[0] != B or kv.seq_lens.shape != (B,):
        raise LayoutError("page_table must be (B, max_pages), seq_lens (B,)")
    lens = kv.seq_lens.long()
    if (lens < 0).any() or (lens > kv.page_table.shape[1] * S).any():
        raise LayoutError("seq_lens out of range for the page table")
    for b in range(B):
        ids = kv.page_table[b, : int((lens[b] + S - 1) // S)].long()
        if ((ids < 0) | (ids >= P)).any():
            raise LayoutError(f"sequence {b} references a page outside [0, {P})")


def unpack_vectorized(packed: torch.Tensor, bit_width: int, head_dim: int) -> torch.Tensor:
    """Same result as `unpack`, as multithreaded torch ops (used where the
    attention operators are timed): index i is read from the two bytes that
    hold stream bits [i*bw, (i+1)*bw)."""
    if bit_width == 8:
        return packed
    if bit_width == 4:                      # byte i = code 2i | code 2i+1 << 4
        return torch.stack((packed & 0x0F, packed >> 4), dim=-1).flatten(-2)
    nb = packed.shape[-1]
    bit = torch.arange(head_dim, dtype=torch.int64) * bit_width
    first, shift = bit // 8, (bit % 8).to(torch.int32)
    second = torch.clamp(first + 1, max=nb - 1)
    words = packed.to(torch.int32)
    lo = words.index_select(-1, first)
    hi = words.index_select(-1, second)
    return (((lo | (hi << 8)) >> shift) & ((1 << bit_width) - 1)).to(torch.uint8)


def _codebook_rows(pages, centroids, bits, D):
    idx = unpack_vectorized(pages, bits, D)
    return centroids.index_select(0, idx.reshape(-1).to(torch.int32)).view(idx.shape)


def _history(kv: OracleKV, b: int):
    """Centroid rows and norms of sequence b in token order: (Hkv, L, D), (Hkv, L)."""
    L, S, D = int(kv.seq_lens[b]), kv.page_size, kv.head_dim
    ids = kv.page_table[b, : -(-L // S)].long()
    def rows(pages, norms, cent, bits):
        p = pages[ids].permute(1, 0, 2, 3).reshape(pages.shape[1], -1, pages.shape[3])[:, :L]
        n = norms[ids].permute(1, 0, 2).reshape(norms.shape[1], -1)[:, :L]
        return _codebook_rows(p, cent, bits, D), n.float()
    return rows(kv.k_pages, kv.k_norms, kv.k_centroids, kv.k_bits), \
        rows(kv.v_pages, kv.v_norms, kv.v_centroids, kv.v_bits)


def reconstruct_attention(q: torch.Tensor, kv: OracleKV, scale: float) -> torch.Tensor:
    """Dequantize each sequence, then causal softmax attention.  (B,Hq,Q,D) fp32."""
    check_layout(q, kv)
    B, Hq, Q, D = q.shape
    rep = Hq // kv.num_kv_heads
    out = torch.zeros(B, Hq, Q, D)
    for b in range(B):
        L = int(kv.seq_lens[b])
        if L == 0:
            continue
        (ck, nk), (cv, nv) = _history(kv, b)
        K = ((ck @ kv.k_Pi) * nk[..., None]).repeat_interleave(rep, 0)   # (Hq, L, D)
        V = ((cv @ kv.v_Pi) * nv[..., None]).repeat_interleave(rep, 0)
        s = (q[b].float() @ K.transpose(1, 2)) * scale                   # (Hq, Q, L)
        last_visible = L - Q + torch.arange(Q)
        hidden = torch.arange(L)[None, :] > last_visible[:, None]        # (Q, L)
        s = s.masked_fill(hidden[None], float("-inf"))
        w = torch.softmax(s, -1).nan_to_num(0.0)
        out[b] = (w @ V) * (~hidden).any(-1)[None, :, None]
    return out


def merge_states(a, b):
    """Combine two online-softmax states (m, l, acc) over disjoint key sets."""
    (m1, l1, a1), (m2, l2, a2) = a, b
    m = torch.maximum(m1, m2)
    w1 = torch.where(torch.isneginf(m1), torch.zeros_like(m1), torch.exp(m1 - m))
    w2 = torch.where(torch.isneginf(m2), torch.zeros_like(m2), torch.exp(m2 - m))
    return m, w1 * l1 + w2 * l2, w1[..., None] * a1 + w2[..., None] * a2


def tiled_attention(q: torch.Tensor, kv: OracleKV, scale: float,
                    split_pages: int | None = None, mutant: str | None = None) -> torch.Tensor:
    """Compressed-domain attention, one page slot at a time, online softmax.

    `mutant` plants one of the reference suite's schedule mistakes
    (turboquant_kv/test_packed_attention.py:246-264) for detection-power tests:
    "update_without_rescale" keeps the old state unscaled when the running
    maximum moves, "merge_without_rescale" adds split states as if they shared
    one maximum.

    q is rotated into the key basis once (q Pi_K^T, times scale); each page
    contributes scores n_K (q_rot . c_K) and values p n_V c_V accumulated in
    the value basis; the result is normalised and rotated back by Pi_V.  With
    `split_pages`, page slots are processed in independent chunks whose states
    are merged afterwards, as a split-K kernel does.  Rows that see no key
    return exact zeros.
    """
    check_layout(q, kv)
    B, Hq, Q, D = q.shape
    S, P = kv.page_size, kv.k_pages.shape[0]
    rep = Hq // kv.num_kv_heads
    head_of = torch.arange(Hq) // rep
    q_rot = (q.float() @ kv.k_Pi.T) * scale
    last_visible = kv.seq_lens.long()[:, None] - Q + torch.arange(Q)[None, :]   # (B, Q)
    slots = kv.page_table.shape[1]
    step = split_pages or slots
    states = []
    for lo in range(0, slots, step):
        m = torch.full((B, Hq, Q), float("-inf"))
        l = torch.zeros(B, Hq, Q)
        acc = torch.zeros(B, Hq, Q, D)
        for t in range(lo, min(lo + step, slots)):
            ids = kv.page_table[:, t].long().clamp(0, P - 1)
            ck = _codebook_rows(kv.k_pages[ids], kv.k_centroids, kv.k_bits, D)[:, head_of]
            cv = _codebook_rows(kv.v_pages[ids], kv.v_centroids, kv.v_bits, D)[:, head_of]
            nk = kv.k_norms[ids].float()[:, head_of]
            nv = kv.v_norms[ids].float()[:, head_of]
            s = (q_rot @ ck.transpose(-1, -2)) * nk[:, :, None, :]               # (B,Hq,Q,S)
            pos = t * S + torch.arange(S)
            hidden = pos[None, None, :] > last_visible[:, :, None]               # (B,Q,S)
            s = s.masked_fill(hidden[:, None], float("-inf"))
            m_new = torch.maximum(m, s.amax(-1))
            alpha = torch.where(torch.isneginf(m), torch.zeros_like(m), torch.exp(m - m_new))
            if mutant == "update_without_rescale":
                alpha = torch.ones_like(alpha)
            p = torch.where(torch.isneginf(s), torch.zeros_like(s), torch.exp(s - m_new[..., None]))
            l = alpha * l + p.sum(-1)
            acc = alpha[..., None] * acc + (p * nv[:, :, None, :]) @ cv
            m = m_new
        states.append((m, l, acc))
    m, l, acc = states[0]
    for st in states[1:]:
        if mutant == "merge_without_rescale":
            m, l, acc = torch.maximum(m, st[0]), l + st[1], acc + st[2]
        else:
            m, l, acc = merge_states((m, l, acc), st)
    a = torch.where(l[..., None] > 0, acc / l.clamp(min=1e-30)[..., None], torch.zeros(()))
    return a @ kv.v_Pi


def default_scale(head_dim: int) -> float:
    return 1.0 / math.sqrt(head_dim)
