"""Data model and contract of attention over paged packed K/V.

A cached head vector x is stored as n = |x| (fp16) and the Lloyd-Max codes of
(x / n) Pi^T.  Since Pi is orthogonal, q . k_hat = n_K (q Pi_K^T) . c_K and
sum_j p_j v_hat_j = (sum_j p_j n_V,j c_V,j) Pi_V: the query is rotated once,
keys and values are read as codes, the output is rotated back once
(reference: turboquant_kv/packed_attention.py:1-43).

    k_pages, v_pages   (P, Hkv, S, NB) uint8    NB = D*bw/8, K and V may differ
    k_norms, v_norms   (P, Hkv, S)     fp16
    page_table         (B, max_pages)  int32    page ids in sequence order, -1 unused
    seq_lens           (B,)            int32    tokens stored per sequence

Query head h reads kv head h // (Hq // Hkv).  The operator itself is
`packed_attention_cuda.packed_decode_attention`.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import _lib
from .packing import packed_bytes


class UnsupportedLayout(ValueError):
    """Raised before any launch when inputs violate the operator contract."""


@dataclass(frozen=True)
class Quantizer:
    """The parts of a `TurboQuantMSE` the attention operator reads."""

    Pi: torch.Tensor          # (D, D) fp32, orthogonal
    centroids: torch.Tensor   # (2**bw,) fp32
    bit_width: int

    @classmethod
    def from_tq(cls, tq) -> "Quantizer":
        return cls(tq.Pi, tq.centroids, tq.bit_width)


@dataclass
class PackedKV:
    """One layer's paged packed K/V and the batch's view of it."""

    k_pages: torch.Tensor
    k_norms: torch.Tensor
    v_pages: torch.Tensor
    v_norms: torch.Tensor
    page_table: torch.Tensor
    seq_lens: torch.Tensor
    k_quant: Quantizer
    v_quant: Quantizer
    head_dim: int

    @property
    def page_size(self) -> int:
        return self.k_pages.shape[2]

    @property
    def num_kv_heads(self) -> int:
        return self.k_pages.shape[1]


@dataclass
class DenseKV:
    """Unquantized paged K/V: pages (P, Hkv, S, D) in the model dtype."""

    k_pages: torch.Tensor
    v_pages: torch.Tensor
    page_table: torch.Tensor
    seq_lens: torch.Tensor
    head_dim: int

    @property
    def page_size(self) -> int:
        return self.k_pages.shape[2]

    @property
    def num_kv_heads(self) -> int:
        return self.k_pages.shape[1]


def check_contract(q: torch.Tensor, kv: PackedKV, *, check_page_ids: bool = True) -> None:
    """Reject what the operators do not support, naming the reason
    (reference: turboquant_kv/packed_attention.py:114-163).

    All checks read metadata only, except the last two (sequence lengths and
    the ids of the pages in use), which copy `seq_lens` and `page_table` to the
    host and therefore wait for the stream.  Callers that built the table
    themselves from validated page references pass `check_page_ids=False`; the
    kernels then still refuse to follow an id outside the pool and say so in
    their status word.
    """
    if q.dim() != 4:
        raise UnsupportedLayout(f"q must be (B, Hq, Q, D), got {tuple(q.shape)}")
    B, Hq, _, D = q.shape
    if D != kv.head_dim:
        raise UnsupportedLayout(f"q head_dim {D} != cache head_dim {kv.head_dim}")
    for side, quant in (("k", kv.k_quant), ("v", kv.v_quant)):
        if tuple(quant.Pi.shape) != (D, D) or quant.Pi.dtype != torch.float32:
            raise UnsupportedLayout(f"{side} rotation must be fp32 ({D}, {D})")
        if quant.centroids.dtype != torch.float32 or quant.centroids.numel() != 2 ** quant.bit_width:
            raise UnsupportedLayout(f"{side} codebook must be fp32 with 2**bw entries")
    try:
        nb_k = packed_bytes(D, kv.k_quant.bit_width)
        nb_v = packed_bytes(D, kv.v_quant.bit_width)
    except ValueError as exc:
        raise UnsupportedLayout(str(exc)) from None
    if kv.k_pages.dim() != 4 or kv.v_pages.dim() != 4:
        raise UnsupportedLayout("pages must be (P, Hkv, S, NB)")
    P, Hkv, S = kv.k_pages.shape[:3]
    if kv.k_pages.dtype != torch.uint8 or kv.v_pages.dtype != torch.uint8:
        raise UnsupportedLayout("packed pages must be uint8")
    if tuple(kv.k_pages.shape) != (P, Hkv, S, nb_k) or tuple(kv.v_pages.shape) != (P, Hkv, S, nb_v):
        raise UnsupportedLayout(
            f"page shapes {tuple(kv.k_pages.shape)}/{tuple(kv.v_pages.shape)} do not match "
            f"(P, Hkv, S, NB) with NB={nb_k}/{nb_v}")
    if tuple(kv.k_norms.shape) != (P, Hkv, S) or tuple(kv.v_norms.shape) != (P, Hkv, S):
        raise UnsupportedLayout("norms must be (P, Hkv, S)")
    if kv.k_norms.dtype != torch.float16 or kv.v_norms.dtype != torch.float16:
        raise UnsupportedLayout("norms must be fp16")
    if Hq % Hkv:
        raise UnsupportedLayout(f"Hq={Hq} is not a multiple of Hkv={Hkv}")
    if kv.page_table.dim() != 2 or kv.page_table.shape[0] != B:
        raise UnsupportedLayout("page_table must be (B, max_pages)")
    if tuple(kv.seq_lens.shape) != (B,):
        raise UnsupportedLayout("seq_lens must be (B,)")
    if kv.page_table.dtype != torch.int32 or kv.seq_lens.dtype != torch.int32:
        raise UnsupportedLayout("page_table and seq_lens must be int32")
    devices = {t.device for t in (q, kv.k_pages, kv.v_pages, kv.k_norms, kv.v_norms,
                                  kv.page_table, kv.seq_lens, kv.k_quant.Pi, kv.v_quant.Pi,
                                  kv.k_quant.centroids, kv.v_quant.centroids)}
    if len(devices) != 1:
        raise UnsupportedLayout(f"all operands must share a device, got {devices}")
    if not check_page_ids:
        return
    lens = kv.seq_lens.to("cpu", torch.int64)
    if bool((lens < 0).any()) or bool((lens > kv.page_table.shape[1] * S).any()):
        raise UnsupportedLayout("seq_lens out of range for the page table")
    table = kv.page_table.to("cpu", torch.int64)
    in_use = torch.arange(table.shape[1])[None, :] < ((lens + S - 1) // S)[:, None]
    bad = in_use & ((table < 0) | (table >= P))
    if bool(bad.any()):
        b = int(bad.any(1).nonzero()[0])
        raise UnsupportedLayout(f"sequence {b} references a page outside [0, {P})")


def kv_head_for(q_head: torch.Tensor, n_rep: int) -> torch.Tensor:
    """Query head -> kv head under grouped-query attention (repeat_kv order)."""
    return q_head // n_rep


def default_scale(head_dim: int) -> float:
    return 1.0 / math.sqrt(head_dim)


def rotate_query(q: torch.Tensor, Pi: torch.Tensor) -> torch.Tensor:
    """Row vector q into the quantizer basis: q Pi^T
    (reference: turboquant_kv/packed_attention.py:173-175)."""
    return q @ Pi.T


def rotate_output(a_rot: torch.Tensor, Pi: torch.Tensor) -> torch.Tensor:
    """Row vector in the quantizer basis back to the model basis: a Pi
    (reference: turboquant_kv/packed_attention.py:178-180)."""
    return a_rot @ Pi


def _safe_exp(x: torch.Tensor, m: torch.Tensor) -> torch.Tensor:
    """exp(x - m) with exp(-inf - -inf) defined as 0."""
    return torch.where(torch.isneginf(m) | torch.isneginf(x), torch.zeros_like(x), torch.exp(x - m))


def merge_partials(left, right):
    """Combine two online-softmax states (m, l, a) covering disjoint key ranges
    (reference: turboquant_kv/packed_attention.py:328-334)."""
    m1, l1, a1 = left
    m2, l2, a2 = right
    m = torch.maximum(m1, m2)
    w1, w2 = _safe_exp(m1, m), _safe_exp(m2, m)
    return m, w1 * l1 + w2 * l2, w1[..., None] * a1 + w2[..., None] * a2


def _require_cuda(q: torch.Tensor, what: str) -> None:
    if not q.is_cuda:
        raise UnsupportedLayout(f"{what}: this package has no CPU implementation; "
                                "operands must be CUDA tensors")


def _causal_rows(q: torch.Tensor, kv: PackedKV):
    """A chunk of Q query tokens as B * Q one-token sequences over the same
    pages: query i of sequence b sits at position seq_lens[b] - Q + i (the
    cache already holds the chunk) and sees the seq_lens[b] - (Q - 1 - i) keys
    up to itself (reference: `_causal_limit`,
    turboquant_kv/packed_attention.py:203-211)."""
    B, Hq, Q, D = q.shape
    rows = q.permute(0, 2, 1, 3).reshape(B * Q, Hq, 1, D)
    if Q == 1:
        return rows, kv
    back = torch.arange(Q - 1, -1, -1, device=kv.seq_lens.device, dtype=torch.int32)
    lens = (kv.seq_lens[:, None] - back[None, :]).clamp_(min=0).reshape(B * Q).contiguous()
    table = kv.page_table.repeat_interleave(Q, dim=0).contiguous()
    return rows, PackedKV(kv.k_pages, kv.k_norms, kv.v_pages, kv.v_norms, table, lens,
                          kv.k_quant, kv.v_quant, kv.head_dim)


def tiled_compressed_attention(q: torch.Tensor, kv: PackedKV, scale: float,
                               split_pages: int | None = None, *,
                               check_page_ids: bool = True) -> torch.Tensor:
    """Causal attention of (B, Hq, Q, D) queries over the packed pages, fp32
    result, on the split-K page-scan kernels: the schedule of the reference's
    operator of this name (turboquant_kv/packed_attention.py:260-311: online
    softmax in the quantizer bases, one rotation of q and one of the output,
    rows that see no key return exact zeros) run on the GPU.  A chunk of Q > 1
    query tokens is one launch over B * Q rows that share the pages, each with
    its own causal length: prefill over packed pages without reconstructing the
    history.  `split_pages` (pages per split, as in the reference) fixes the
    split-K factor; None lets the backend choose.  `check_page_ids=False`
    (additive) skips the host-side check of lengths and page ids, which waits
    for the stream, when the table comes from validated page references."""
    check_contract(q, kv, check_page_ids=check_page_ids)
    _require_cuda(q, "tiled_compressed_attention")
    from .packed_attention_cuda import (packed_decode_attention, packed_prefill_attention,
                                        prefill_supported)
    B, Hq, Q, D = q.shape
    if Q > 1 and prefill_supported(q, kv):
        # one pass over the pages for the whole chunk (wtq_prefill)
        splits = None if not split_pages else max(1, -(-kv.page_table.shape[1] // int(split_pages)))
        return packed_prefill_attention(q.float(), kv, scale, num_splits=splits,
                                        check_page_ids=False).contiguous()
    rows, view = _causal_rows(q.float(), kv)
    splits = None if not split_pages else max(1, -(-kv.page_table.shape[1] // int(split_pages)))
    out = packed_decode_attention(rows.contiguous(), view, scale, num_splits=splits,
                                  check_page_ids=False)
    return out.view(B, Q, Hq, D).permute(0, 2, 1, 3).contiguous()


def explicit_compressed_attention(q: torch.Tensor, kv: PackedKV, scale: float) -> torch.Tensor:
    """The reference's single-softmax form of the same algebra
    (turboquant_kv/packed_attention.py:238-257).  On the GPU there is one
    schedule for it: this is `tiled_compressed_attention` with one split."""
    return tiled_compressed_attention(q, kv, scale, split_pages=kv.page_table.shape[1])


def reconstruct_attention(q: torch.Tensor, kv: PackedKV, scale: float) -> torch.Tensor:
    """Dequantize every sequence's history (fused unpack, gather, rotate and
    scale kernel), then plain causal attention in fp32 on the same device: the
    independent check of the compressed-domain operators
    (reference: turboquant_kv/packed_attention.py:214-235)."""
    check_contract(q, kv)
    _require_cuda(q, "reconstruct_attention")
    from .cache import dequantize_rows
    B, Hq, Q, D = q.shape
    S = kv.page_size
    n_rep = Hq // kv.num_kv_heads
    out = torch.zeros(B, Hq, Q, D, dtype=torch.float32, device=q.device)
    lens = kv.seq_lens.tolist()
    heads = kv_head_for(torch.arange(Hq, device=q.device), n_rep)
    pos = torch.arange(Q, device=q.device)
    for b, L in enumerate(lens):
        if L <= 0:
            continue
        ids = kv.page_table[b, :(L + S - 1) // S].long()
        sides = []
        for pages, norms, quant in ((kv.k_pages, kv.k_norms, kv.k_quant),
                                    (kv.v_pages, kv.v_norms, kv.v_quant)):
            rows = pages[ids].permute(1, 0, 2, 3).reshape(pages.shape[1], -1, pages.shape[3])[:, :L]
            nrm = norms[ids].permute(1, 0, 2).reshape(norms.shape[1], -1)[:, :L]
            rows = rows.contiguous()
            full = torch.empty(*rows.shape[:-1], D, dtype=torch.float32, device=q.device)
            sides.append(dequantize_rows(rows, nrm.contiguous(), quant.centroids, quant.Pi,
                                         quant.bit_width, D, out=full)[heads])
        k, v = sides                                                  # (Hq, L, D)
        s = (q[b].float() @ k.transpose(-1, -2)) * scale             # (Hq, Q, L)
        limit = L - Q + pos                                           # last key query i may see
        allowed = torch.arange(L, device=q.device)[None, :] <= limit[:, None]
        s = s.masked_fill(~allowed[None], float("-inf"))
        p = torch.softmax(s, dim=-1).nan_to_num(0.0)
        out[b] = (p @ v) * allowed.any(-1)[None, :, None]
    return out


@torch.no_grad()
def pages_from_dense(k: torch.Tensor, v: torch.Tensor, seq_lens, k_tq, v_tq, page_size: int,
                     num_pages: int | None = None,
                     generator: torch.Generator | None = None) -> PackedKV:
    """Quantize dense (B, Hkv, Lmax, D) CUDA K/V into randomly ordered pages.

    Fixture builder with the reference's page assignment
    (turboquant_kv/packed_attention.py:341-377): ids come from one
    `torch.randperm(total, generator)` (CPU generator) consumed in (sequence,
    page) order; unused table slots hold -1.  Every full page of a sequence is
    quantized in one launch; a short tail of 2..5 vectors gets its own launch so
    that its rotation uses the summation order the reference's CPU arithmetic
    uses for a call that small.
    """
    dev = _lib.require_cuda(k, v)
    B, Hkv, _, D = k.shape
    lens = [int(x) for x in seq_lens]
    need = [-(-L // page_size) for L in lens]
    total = num_pages or max(sum(need), 1)
    order = torch.randperm(total, generator=generator)
    nb_k, nb_v = packed_bytes(D, k_tq.bit_width), packed_bytes(D, v_tq.bit_width)
    kp = torch.zeros(total, Hkv, page_size, nb_k, dtype=torch.uint8, device=dev)
    vp = torch.zeros(total, Hkv, page_size, nb_v, dtype=torch.uint8, device=dev)
    kn = torch.zeros(total, Hkv, page_size, dtype=torch.float16, device=dev)
    vn = torch.zeros(total, Hkv, page_size, dtype=torch.float16, device=dev)
    table = torch.full((B, max(max(need), 1)), -1, dtype=torch.int32)
    at = 0
    for b in range(B):
        table[b, :need[b]] = order[at:at + need[b]].to(torch.int32)
        at += need[b]
    table_dev = table.to(dev)
    for b, L in enumerate(lens):
        if L == 0:
            continue
        ids = table_dev[b, :need[b]].long()
        full = L // page_size                 # pages filled completely
        tail = L - full * page_size
        # (first token, last token + 1, vectors per reference call): the
        # reference quantizes one (sequence, page) slab of Hkv x tokens vectors
        # per call, and 2..5 vectors in a call select the interleaved order.
        spans = []
        if full:
            if not 2 <= Hkv * page_size <= 5:
                spans.append((0, full * page_size, Hkv * page_size))
            else:
                spans += [(t * page_size, (t + 1) * page_size, Hkv * page_size)
                          for t in range(full)]
        if tail:
            spans.append((full * page_size, L, Hkv * tail))
        for dense, tq, pages, norms in ((k, k_tq, kp, kn), (v, v_tq, vp, vn)):
            for lo, hi, call_rows in spans:
                mode = _lib.ORDER_INTERLEAVED16 if 2 <= call_rows <= 5 else _lib.ORDER_SEQUENTIAL
                codes, nrm = tq.quantize(dense[b, :, lo:hi], order=mode, packed=True)
                n_tok, first = hi - lo, lo // page_size
                if n_tok % page_size == 0:            # whole pages: (Hkv, pages*S, NB)
                    n_pg = n_tok // page_size
                    dst = ids[first:first + n_pg]
                    pages[dst] = codes.view(Hkv, n_pg, page_size, -1).permute(1, 0, 2, 3)
                    norms[dst] = nrm.to(torch.float16).view(Hkv, n_pg, page_size).permute(1, 0, 2)
                else:
                    pages[ids[first], :, :n_tok] = codes
                    norms[ids[first], :, :n_tok] = nrm.to(torch.float16)
    return PackedKV(kp, kn, vp, vn, table_dev,
                    torch.tensor(lens, dtype=torch.int32, device=dev),
                    Quantizer.from_tq(k_tq), Quantizer.from_tq(v_tq), D)
