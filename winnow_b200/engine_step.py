"""One decode step of a fixed batch, layer by layer, with everything the kernels
need resident on the device and every launch marshalled once.

The reference's engine builds a fresh cache object per forward, rebuilds the
page table on the host, copies it to the device and, in every layer, reads it
back to compute page ids (turboquant_kv/engine.py:183-195,
turboquant_kv/packed_backend.py:114-170).  Here a `DecodeSession` is created
when the batch composition changes and then lives for many steps:

* the page table is a `DeviceTable` (rows rewritten only when a sequence crosses
  a page boundary), the lengths are an int32 tensor advanced on the device;
* each layer owns one `AppendPlan` and one `DecodePlan` over fixed staging
  tensors (`k_in`, `v_in`, `q_in`, `out`), so a layer's append + attention is two
  library calls with no Python-side checks, or, after `capture()`, the replay
  of one CUDA graph holding both;
* one status word collects what the kernels refused (a page id outside the
  pool, a position outside the table); `check()` raises if it is non-zero.

The model's projections write K, V and the query of the new token straight into
the staging tensors (or pass them to `layer()`, which copies); `out` holds the
attention result of the layer just run.  Page ownership, reservation and fenced
release stay with the `PagePool`, exactly as for `PagedPackedCache`.
"""
from __future__ import annotations

import torch

from . import _lib
from . import packed_attention as pa
from .packed_attention_cuda import DecodePlan, decode_workspace
from .packed_backend import AppendPlan
from .page_pool import DeviceTable, PagePool, StalePage


class DecodeSession:
    def __init__(self, pool: PagePool, owners, lengths, *, k_quant, v_quant, head_dim: int,
                 q_heads: int, dtype: torch.dtype, max_tokens: int, scale: float | None = None,
                 num_splits: int | None = None):
        """`lengths[b]`: tokens sequence b already stores; `max_tokens`: the
        longest any sequence may get while this session lives (fixes the table
        width, hence the split-K plan)."""
        if pool.dense:
            raise ValueError("DecodeSession serves packed pools")
        dev = pool.device
        if dev.type != "cuda":
            raise _lib.BackendError("DecodeSession needs a pool on a CUDA device; there is no CPU path")
        self.pool, self.owners = pool, list(owners)
        self.lengths = [int(x) for x in lengths]
        B, Hkv, D = len(self.owners), pool.num_kv_heads, head_dim
        self.scale = float(scale if scale is not None else D ** -0.5)
        self.table = DeviceTable(pool, self.owners, max(1, pool.pages_for(max_tokens)), dev)
        self.max_tokens = self.table.width * pool.page_size
        self.seq = torch.tensor(self.lengths, dtype=torch.int32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.k_in = torch.zeros(B, Hkv, 1, D, dtype=dtype, device=dev)
        self.v_in = torch.zeros(B, Hkv, 1, D, dtype=dtype, device=dev)
        self.q_in = torch.zeros(B, q_heads, 1, D, dtype=dtype, device=dev)
        self.out = torch.zeros(B, q_heads, 1, D, dtype=dtype, device=dev)
        self.table.refresh(self.lengths)
        ws = decode_workspace(B, q_heads, Hkv, D, self.table.width, pool.page_size,
                              int(num_splits or 0), dev)
        kq, vq = pa.Quantizer.from_tq(k_quant), pa.Quantizer.from_tq(v_quant)
        self._append, self._decode = [], []
        for layer in range(pool.num_layers):
            kv = pa.PackedKV(pool.k_pages[layer], pool.k_norms[layer], pool.v_pages[layer],
                             pool.v_norms[layer], self.table.table, self.seq, kq, vq, D)
            self._append.append(AppendPlan(self.k_in, self.v_in, kv.k_pages, kv.k_norms, kv.v_pages,
                                           kv.v_norms, self.table.table, self.seq, k_quant, v_quant,
                                           status=self.status))
            # (page ids come from the pool's own reservations: no per-call host check)
            self._decode.append(DecodePlan(self.q_in, kv, self.scale, num_splits=num_splits,
                                           out=self.out, workspace=ws, status=self.status,
                                           check_page_ids=False))
        self._graphs = None
        self._one = torch.ones((), dtype=torch.int32, device=dev)

    # ---- step protocol -----------------------------------------------------------
    def begin_step(self) -> None:
        """Reserve room for one more token per sequence (all or nothing), bring
        the device table up to date, advance the lengths on the device."""
        want = [L + 1 for L in self.lengths]
        if max(want, default=0) > self.max_tokens:
            raise StalePage(f"a sequence would reach {max(want)} tokens; this session was sized "
                            f"for {self.max_tokens}")
        self.pool.ensure_many(self.owners, want)
        self.table.refresh(want)
        self.seq.add_(self._one)                 # lengths now include the token being appended
        self.lengths = want

    def layer(self, layer_idx: int, k=None, v=None, q=None) -> torch.Tensor:
        """Append the new token's K/V of this layer and attend; returns `out`
        (overwritten by the next layer).  k, v: (B, Hkv, 1, D); q: (B, Hq, 1, D);
        omitted ones are taken from the staging tensors as they are."""
        if k is not None:
            self.k_in.copy_(k)
        if v is not None:
            self.v_in.copy_(v)
        if q is not None:
            self.q_in.copy_(q)
        if self._graphs is not None:
            self._graphs[layer_idx].replay()
        else:
            self._append[layer_idx].run()
            self._decode[layer_idx].run()
        return self.out

    def capture(self) -> None:
        """Capture each layer's append + attention as one CUDA graph.  The calls
        made while capturing are real ones: they write the staging tensors'
        present content into the position the current step appends to, in every
        layer.  Call it right after a `begin_step()`, before that step's
        `layer()` calls: those then overwrite the same slots with the real
        token, layer by layer, before anything reads them."""
        dev = self.pool.device
        with torch.cuda.device(dev):
            for a, d in zip(self._append, self._decode):      # one-time set-up outside capture
                a.run()
                d.run()
            torch.cuda.synchronize()
            graphs = []
            for a, d in zip(self._append, self._decode):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    a.run()
                    d.run()
                graphs.append(g)
        self._graphs = graphs

    def check(self) -> None:
        """Raise if a kernel refused a page id or a position since the last
        check (synchronises; call where the loop syncs anyway, e.g. before
        sampling)."""
        word = int(self.status.item())
        if word:
            self.status.zero_()
            raise StalePage(f"decode step: the kernels refused part of the batch (status {word:#x}: "
                            f"bit {_lib.STATUS_BAD_PAGE} page id outside the pool, bit "
                            f"{_lib.STATUS_BAD_POSITION} position outside the page table)")
