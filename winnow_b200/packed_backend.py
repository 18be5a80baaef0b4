"""Transformers integration: a cache that appends into packed pages and an
attention function that reads them, both on the CUDA backend.

`PagedPackedCache.update` quantizes the new K/V of one layer straight into the
pool's pages with one fused launch (wtq_append) and hands back a `PackedKV`
handle instead of tensors.  The attention function registered as
``winnow_packed`` receives that handle as key and value:

* decode (one query token per sequence) runs `packed_decode_attention`; no
  (B, Hkv, L, D) history exists at any point;
* a prefill chunk (several query tokens) dequantizes the one sequence's history
  with the fused dequant kernel and calls SDPA with an offset causal mask, the
  fallback the reference documents for that case.

Mirrors turboquant_kv/packed_backend.py (entry points, names, error behaviour);
what differs: the page table and lengths stay on the device (no per-layer host
round trip), K and V may use different bit widths, and `auto` resolves to the
single backend `cuda_packed` (the name `triton_packed` is kept as an alias).
There is no CPU path: CPU tensors raise.
"""
from __future__ import annotations

import ctypes
from collections import Counter

import torch
import torch.nn.functional as F

from . import _lib
from . import packed_attention as pa
from .cache import _get_quantizer, dequantize_rows
from .packed_attention_cuda import _side, dense_decode_attention, packed_decode_attention
from .packing import packed_bytes
from .page_pool import PagePool, StalePage

ATTN_NAME = "winnow_packed"
SUPPORTED_ARCH = ("Qwen2ForCausalLM", "LlamaForCausalLM")

# Attention calls served per backend; tests and studies read this to prove
# which path ran.
BACKEND_COUNTS: Counter = Counter()

DECODE_BACKENDS = ("auto", "cuda_packed", "triton_packed", "reconstruct_sdpa")


class UnsupportedModel(ValueError):
    pass


def head_dim_of(config) -> int:
    return getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads


def check_model(config, bit_width: int, bit_width_v: int | None = None) -> None:
    arch = (getattr(config, "architectures", None) or ["?"])[0]
    if arch not in SUPPORTED_ARCH:
        raise UnsupportedModel(f"{arch} is not a supported architecture {SUPPORTED_ARCH}")
    if getattr(config, "use_sliding_window", False):
        raise UnsupportedModel("sliding-window attention is not supported")
    kinds = set(getattr(config, "layer_types", None) or ["full_attention"])
    if kinds != {"full_attention"}:
        raise UnsupportedModel(f"layer types {sorted(kinds)} are not all full attention")
    D = head_dim_of(config)
    packed_bytes(D, bit_width)
    packed_bytes(D, bit_width if bit_width_v is None else bit_width_v)


def make_pool(config, *, bit_width: int | None, num_pages: int, page_size: int, device,
              max_pages_per_request=None, fence_factory=None,
              dense_dtype: torch.dtype | None = None, bit_width_v: int | None = None) -> PagePool:
    """Packed pool at `bit_width` (values at `bit_width_v` when given), or with
    `dense_dtype` an unquantized pool."""
    D = head_dim_of(config)
    if dense_dtype is not None:
        nb_k = nb_v = D
    else:
        nb_k = packed_bytes(D, bit_width)
        nb_v = packed_bytes(D, bit_width if bit_width_v is None else bit_width_v)
    return PagePool(num_layers=config.num_hidden_layers, num_pages=num_pages,
                    num_kv_heads=config.num_key_value_heads, page_size=page_size,
                    nb_k=nb_k, nb_v=nb_v, device=device,
                    max_pages_per_request=max_pages_per_request,
                    fence_factory=fence_factory, dense_dtype=dense_dtype)


def quantizers_for(config, bit_width: int, device, k_seed: int = 42, v_seed: int = 42,
                   bit_width_v: int | None = None):
    """K and V quantizers; by default both use rotation seed 42 like the
    reference's contiguous cache, so both store identical bytes."""
    D = head_dim_of(config)
    return (_get_quantizer(bit_width, D, device, seed=k_seed),
            _get_quantizer(bit_width if bit_width_v is None else bit_width_v, D, device, seed=v_seed))


class PagedPackedCache:
    """Cache object for one forward over a batch of pool-backed sequences.

    `owners[b]` is the request whose pages hold sequence b and `lengths[b]` the
    tokens it already stores.  The forward appends the same number of tokens n
    to every sequence (1 in batched decode, the chunk length in prefill).
    Lengths advance after the last layer has written.
    """

    def __init__(self, pool: PagePool, owners, lengths, *, k_quant, v_quant, head_dim: int,
                 decode_backend: str = "auto", prefill_backend: str = "auto"):
        """`prefill_backend` (additive keyword): "packed" runs a chunk of query
        tokens on the packed pages (the chunk kernel `wtq_prefill` where the
        layout allows, B * Q decode rows otherwise: no reconstruction);
        "reconstruct" is the reference's path (dequantize the history, stock
        attention); "auto" picks "packed" where the chunk kernel serves the
        layout and "reconstruct" elsewhere."""
        if prefill_backend not in ("auto", "reconstruct", "packed"):
            raise ValueError(f"unknown prefill_backend {prefill_backend!r}")
        self.prefill_backend = prefill_backend
        self.pool = pool
        self.owners = list(owners)
        self.lengths = list(lengths)
        self.kq, self.vq = k_quant, v_quant
        self.head_dim = head_dim
        self.decode_backend = decode_backend
        self._table = self._seq = self._refs = None
        self.status = None

    def get_seq_length(self, layer_idx: int = 0) -> int:
        if len(set(self.lengths)) != 1:
            raise RuntimeError("mixed lengths: pass explicit position_ids")
        return self.lengths[0]

    def check(self) -> None:
        """Raise `StalePage` if a kernel of this forward refused a page id or a
        position (it skipped the access and set a bit in `self.status`, which
        both the append and the attention launches report into).  Synchronises:
        call it where the caller syncs anyway, e.g. before sampling."""
        if self.status is None:
            return
        word = int(self.status.item())
        if word:
            self.status.zero_()
            raise StalePage(f"forward refused part of the batch (status {word:#x}: bit "
                            f"{_lib.STATUS_BAD_PAGE} page id outside the pool, bit "
                            f"{_lib.STATUS_BAD_POSITION} position outside the page table)")

    def _prepare(self, n: int, device):
        """Once per forward: check ownership and reservation, build the page
        table and the post-append lengths, and copy both to the device.  Never
        allocates pages: a forward racing a release must fail."""
        refs = [self.pool.held(o) for o in self.owners]
        for owner, held, L in zip(self.owners, refs, self.lengths):
            if self.pool.pages_for(L + n) > len(held):
                raise StalePage(f"{owner} holds {len(held)} pages, needs {self.pool.pages_for(L + n)}")
            self.pool.validate(owner, held)
        width = max(max((len(r) for r in refs), default=0), 1)
        table = torch.full((len(refs), width), -1, dtype=torch.int32)
        for b, held in enumerate(refs):
            if held:
                table[b, :len(held)] = torch.tensor([r.page for r in held], dtype=torch.int32)
        self._refs = refs
        self._table = table.to(device, non_blocking=True)
        self._seq = torch.tensor([L + n for L in self.lengths], dtype=torch.int32).to(
            device, non_blocking=True)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)

    @torch.no_grad()
    def update(self, key_states, value_states, layer_idx, *args, **kwargs):
        B, Hkv, n, D = key_states.shape
        if B != len(self.owners):
            raise RuntimeError(f"batch {B} != {len(self.owners)} owners")
        dev = _lib.require_cuda(key_states, value_states, self.pool.k_pages)
        if layer_idx == 0 or self._table is None:
            self._prepare(n, dev)
        pool = self.pool
        last = layer_idx == pool.num_layers - 1
        if pool.dense:
            S = pool.page_size
            pos = torch.tensor([[L + i for i in range(n)] for L in self.lengths], device=dev)
            pids = torch.gather(self._table.long(), 1, pos // S)
            slots = pos % S
            for src, pages in ((key_states, pool.k_pages), (value_states, pool.v_pages)):
                pages[layer_idx][pids, :, slots] = src.permute(0, 2, 1, 3).to(pages.dtype)
            handle = pa.DenseKV(pool.k_pages[layer_idx], pool.v_pages[layer_idx],
                                self._table, self._seq, D)
        else:
            append_tokens(key_states, value_states, pool.k_pages[layer_idx], pool.k_norms[layer_idx],
                          pool.v_pages[layer_idx], pool.v_norms[layer_idx], self._table, self._seq,
                          self.kq, self.vq, status=self.status)
            handle = pa.PackedKV(pool.k_pages[layer_idx], pool.k_norms[layer_idx],
                                 pool.v_pages[layer_idx], pool.v_norms[layer_idx],
                                 self._table, self._seq, pa.Quantizer.from_tq(self.kq),
                                 pa.Quantizer.from_tq(self.vq), D)
            handle.table_validated = True      # ids come from validated page refs
        handle.decode_backend = self.decode_backend
        handle.prefill_backend = self.prefill_backend
        handle.status = self.status             # the attention call reports into the same word
        if last:
            self.lengths = [L + n for L in self.lengths]
        return handle, handle


class AppendPlan:
    """One fused append (wtq_append) with every argument checked and marshalled
    ahead of time; `run()` is a single library call on the current stream.  The
    plan keeps its tensors alive and can be reused while they are updated in
    place (new K/V written into the same staging tensors, lengths advanced)."""

    def __init__(self, k, v, k_pages, k_norms, v_pages, v_norms, page_table, seq_lens, k_tq, v_tq,
                 *, order: int = _lib.ORDER_AUTO, status: torch.Tensor | None = None):
        dev = _lib.require_cuda(k, v, k_pages, v_pages, k_norms, v_norms, page_table, seq_lens)
        B, Hkv, n, D = k.shape
        if v.shape != k.shape or v.dtype != k.dtype:
            raise ValueError("k and v must have the same shape and dtype")
        if k.stride(-1) != 1 or v.stride(-1) != 1:
            raise ValueError("k and v need unit stride in their last dimension")
        P, Hp, S, _ = k_pages.shape
        if Hp != Hkv or v_pages.shape[:3] != k_pages.shape[:3]:
            raise ValueError("pages do not match (P, Hkv, S, NB)")
        for pages, norms, tq in ((k_pages, k_norms, k_tq), (v_pages, v_norms, v_tq)):
            if pages.shape[-1] != packed_bytes(D, tq.bit_width) or pages.stride(-1) != 1 \
                    or pages.stride(-2) != pages.shape[-1] or norms.stride(-1) != 1 \
                    or norms.dtype != torch.float16 or pages.dtype != torch.uint8:
                raise ValueError("pages/norms layout does not match the quantizer")
        if page_table.dtype != torch.int32 or seq_lens.dtype != torch.int32 \
                or page_table.stride(-1) != 1 or not seq_lens.is_contiguous():
            raise ValueError("page_table and seq_lens must be contiguous int32")
        self.device = dev
        self._keep = (k, v, k_pages, k_norms, v_pages, v_norms, page_table, seq_lens, k_tq, v_tq, status)
        self._sides = [
            _lib.Side(pages.data_ptr(), norms.data_ptr(), pages.stride(0), pages.stride(1),
                      norms.stride(0), norms.stride(1), tq.Pi.data_ptr(), tq.boundaries.data_ptr(),
                      tq.centroids.data_ptr(), tq.bit_width)
            for pages, norms, tq in ((k_pages, k_norms, k_tq), (v_pages, v_norms, v_tq))]
        self._ks = _lib.i64x(k.stride(0), k.stride(1), k.stride(2))
        self._vs = _lib.i64x(v.stride(0), v.stride(1), v.stride(2))
        self._fn = _lib.lib().wtq_append
        self._args = (k.data_ptr(), v.data_ptr(), _lib.dtype_code(k.dtype), self._ks, self._vs,
                      ctypes.byref(self._sides[0]), ctypes.byref(self._sides[1]),
                      page_table.data_ptr(), page_table.stride(0), seq_lens.data_ptr(),
                      B, Hkv, n, D, S, P, page_table.shape[1], order,
                      status.data_ptr() if status is not None else None)

    def run(self) -> None:
        rc = self._fn(*self._args, torch.cuda.current_stream(self.device).cuda_stream)
        if rc:
            _lib.check(rc)


@torch.no_grad()
def append_tokens(k, v, k_pages, k_norms, v_pages, v_norms, page_table, seq_lens, k_tq, v_tq, *,
                  order: int = _lib.ORDER_AUTO, status: torch.Tensor | None = None) -> None:
    """Fused append of n tokens per sequence into one layer's pages.

    k, v: (B, Hkv, n, D) CUDA tensors (any strides with a contiguous last
    dimension); pages (P, Hkv, S, NB) / norms (P, Hkv, S) of one layer;
    `seq_lens` already includes the n new tokens, so token i of sequence b is
    written at position seq_lens[b] - n + i.
    """
    if k.stride(-1) != 1:
        k = k.contiguous()
    if v.stride(-1) != 1:
        v = v.contiguous()
    plan = AppendPlan(k, v, k_pages, k_norms, v_pages, v_norms, page_table, seq_lens, k_tq, v_tq,
                      order=order, status=status)
    with torch.cuda.device(plan.device):
        plan.run()


def select_decode_backend(query: torch.Tensor, kv, requested: str) -> str:
    """Which operator serves a decode step.  Unsupported requests fail loudly."""
    if isinstance(kv, pa.DenseKV):
        if requested == "dense_sdpa":
            return "dense_sdpa"
        if requested in ("auto", "cuda_dense", "triton_dense"):
            if query.is_cuda:
                _lib.lib()                       # raises if the library is not built
                return "cuda_dense"
            if requested == "auto":
                return "dense_sdpa"
            raise RuntimeError(f"{requested} requested but the query is not on a CUDA device")
        raise ValueError(f"backend {requested!r} does not read dense pages")
    if requested not in DECODE_BACKENDS:
        raise ValueError(f"unknown decode backend {requested!r}")
    if not query.is_cuda:
        raise RuntimeError(f"{requested} requested but the query is not on a CUDA device; "
                           "this build has no CPU backend")
    _lib.lib()                                   # raises if the library is not built
    if requested in ("auto", "cuda_packed", "triton_packed"):
        return "cuda_packed"
    return requested


def dequantize_history(kv: pa.PackedKV, pages, norms, quant, b: int, dtype) -> torch.Tensor:
    """(1, Hkv, L, D) reconstruction of sequence b (prefill fallback)."""
    L = int(kv.seq_lens[b])
    S = kv.page_size
    ids = kv.page_table[b, : -(-L // S)].long()
    rows = pages[ids].permute(1, 0, 2, 3).reshape(pages.shape[1], -1, pages.shape[3])[:, :L]
    nrm = norms[ids].permute(1, 0, 2).reshape(norms.shape[1], -1)[:, :L]
    out = torch.empty(1, rows.shape[0], L, kv.head_dim, dtype=dtype, device=rows.device)
    dequantize_rows(rows.contiguous(), nrm.contiguous(), quant.centroids, quant.Pi,
                    quant.bit_width, kv.head_dim, out=out[0])
    return out


def _offset_causal_mask(L: int, Q: int, device) -> torch.Tensor:
    return torch.arange(L, device=device)[None, :] <= (L - Q + torch.arange(Q, device=device))[:, None]


def _reconstruct_sdpa(query, kv: pa.PackedKV, scaling):
    """Per sequence: dequantize, then SDPA with an offset causal mask."""
    B, Hq, Q, D = query.shape
    out = torch.zeros(B, Hq, Q, D, dtype=query.dtype, device=query.device)
    for b in range(B):
        L = int(kv.seq_lens[b])
        if L == 0:
            continue
        k = dequantize_history(kv, kv.k_pages, kv.k_norms, kv.k_quant, b, query.dtype)
        v = dequantize_history(kv, kv.v_pages, kv.v_norms, kv.v_quant, b, query.dtype)
        out[b] = F.scaled_dot_product_attention(
            query[b:b + 1], k, v, attn_mask=_offset_causal_mask(L, Q, query.device),
            scale=scaling, enable_gqa=Hq != k.shape[1])[0]
    return out


def _dense_sdpa(query, kv: pa.DenseKV, scaling):
    """Per sequence: gather unquantized pages, SDPA with an offset causal mask."""
    B, Hq, Q, D = query.shape
    out = torch.zeros(B, Hq, Q, D, dtype=query.dtype, device=query.device)
    S = kv.page_size
    for b in range(B):
        L = int(kv.seq_lens[b])
        if L == 0:
            continue
        ids = kv.page_table[b, : -(-L // S)].long()

        def history(pages):
            return pages[ids].permute(1, 0, 2, 3).reshape(pages.shape[1], -1, D)[None, :, :L]

        out[b] = F.scaled_dot_product_attention(
            query[b:b + 1], history(kv.k_pages).to(query.dtype), history(kv.v_pages).to(query.dtype),
            attn_mask=_offset_causal_mask(L, Q, query.device), scale=scaling,
            enable_gqa=Hq != kv.num_kv_heads)[0]
    return out


def _prefill_choice(query, kv) -> str:
    """ "packed" or "reconstruct" for a chunk of query tokens over `kv`."""
    want = getattr(kv, "prefill_backend", "reconstruct")
    if want != "auto":
        return want
    from .packed_attention_cuda import prefill_supported
    return "packed" if prefill_supported(query, kv) else "reconstruct"


def winnow_packed_attention(module, query, key, value, attention_mask, dropout: float = 0.0,
                            scaling=None, **kwargs):
    """`AttentionInterface` entry point.  Returns ((B, Q, Hq, D), None)."""
    scaling = scaling if scaling is not None else query.shape[-1] ** -0.5
    if not isinstance(key, (pa.PackedKV, pa.DenseKV)):
        from transformers.integrations.sdpa_attention import sdpa_attention_forward
        BACKEND_COUNTS["native_sdpa"] += 1
        return sdpa_attention_forward(module, query, key, value, attention_mask,
                                      dropout=dropout, scaling=scaling, **kwargs)
    Q = query.shape[2]
    requested = getattr(key, "decode_backend", "auto")
    if isinstance(key, pa.DenseKV):
        backend = "dense_sdpa" if Q > 1 else select_decode_backend(query, key, requested)
        BACKEND_COUNTS[("prefill_" if Q > 1 else "") + backend] += 1
        if Q == 1 and requested == "triton_dense":
            BACKEND_COUNTS["triton_dense"] += 1            # the reference's name, kept as an alias
        if backend == "cuda_dense":
            out = dense_decode_attention(query, key, scaling, num_splits=0)
        else:
            out = _dense_sdpa(query, key, scaling)
    elif Q > 1 and query.is_cuda and _prefill_choice(query, key) == "packed":
        BACKEND_COUNTS["prefill_cuda_packed"] += 1
        from .packed_attention_cuda import packed_prefill_attention, prefill_supported
        check = not getattr(key, "table_validated", False)
        if prefill_supported(query, key):            # the chunk kernel, in the query's dtype
            out = packed_prefill_attention(query, key, scaling, check_page_ids=check)
        else:                                        # B * Q decode rows over the same pages
            out = pa.tiled_compressed_attention(query, key, scaling,
                                                check_page_ids=check).to(query.dtype)
    elif Q > 1:
        BACKEND_COUNTS["prefill_reconstruct_sdpa"] += 1
        out = _reconstruct_sdpa(query, key, scaling)
    else:
        backend = select_decode_backend(query, key, requested)
        BACKEND_COUNTS[backend] += 1
        if requested == "triton_packed":
            BACKEND_COUNTS["triton_packed"] += 1
        if backend == "cuda_packed":
            out = packed_decode_attention(
                query, key, scaling, status=getattr(key, "status", None),
                check_page_ids=not getattr(key, "table_validated", False))
        else:
            out = _reconstruct_sdpa(query, key, scaling)
    return out.transpose(1, 2).contiguous(), None


def register() -> None:
    from transformers import AttentionInterface
    AttentionInterface.register(ATTN_NAME, winnow_packed_attention)
