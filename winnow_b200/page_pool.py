"""Page pool for packed KV: request-scoped ownership and fenced reuse.

Host-side bookkeeping with the semantics of the reference allocator
(turboquant_kv/page_pool.py:62-175); the tensors it owns are what the CUDA
kernels read and write:

    k_pages, v_pages  (layers, P, Hkv, S, NB) uint8   packed codes
    k_norms, v_norms  (layers, P, Hkv, S)     fp16

Page id p means page p of every layer, so a request reserves pages once per
token span.  A page is held under (owner, generation).  Releasing an owner
bumps the generation at once, so launches still holding the old `PageRef`s fail
`validate`; the page itself only returns to the free list when the fence
recorded after the last launch that could read it has completed.  Admission is
all-or-nothing: `ensure` raises `PoolExhausted` and never evicts.
"""
from __future__ import annotations

import threading
from collections import deque
from dataclasses import dataclass

import torch


class PoolExhausted(RuntimeError):
    """Not enough free pages; refuse or queue the request."""


class StalePage(RuntimeError):
    """A launch referenced a page its caller no longer owns."""


@dataclass(frozen=True)
class PageRef:
    page: int
    generation: int


class _Completed:
    """Fence of work that is already finished (CPU bookkeeping only)."""

    def query(self) -> bool:
        return True

    def synchronize(self) -> None:
        return None


def default_fence(device: torch.device):
    """An event recorded now on the device's current stream."""
    if torch.device(device).type != "cuda":
        return _Completed()
    event = torch.cuda.Event()
    event.record(torch.cuda.current_stream(device))
    return event


class PagePool:
    def __init__(self, *, num_layers: int, num_pages: int, num_kv_heads: int, page_size: int,
                 nb_k: int, nb_v: int, device="cpu", max_pages_per_request: int | None = None,
                 fence_factory=None, dense_dtype: torch.dtype | None = None):
        """`nb_k` / `nb_v` are bytes per packed K / V vector and may differ
        (e.g. 4-bit keys with 6-bit values).  With `dense_dtype` the pages hold
        unquantized rows of nb elements of that dtype and there are no norms."""
        self.device = torch.device(device)
        self.num_layers, self.num_pages, self.page_size = num_layers, num_pages, page_size
        self.num_kv_heads = num_kv_heads
        self.dense = dense_dtype is not None
        lead = (num_layers, num_pages, num_kv_heads, page_size)
        store = dense_dtype if self.dense else torch.uint8
        self.k_pages = torch.zeros(*lead, nb_k, dtype=store, device=self.device)
        self.v_pages = torch.zeros(*lead, nb_v, dtype=store, device=self.device)
        if self.dense:
            self.k_norms = self.v_norms = None
        else:
            self.k_norms = torch.zeros(*lead, dtype=torch.float16, device=self.device)
            self.v_norms = torch.zeros(*lead, dtype=torch.float16, device=self.device)
        self.max_pages_per_request = max_pages_per_request or num_pages
        self._make_fence = fence_factory or (lambda: default_fence(self.device))
        self._generation = [0] * num_pages
        self._owner_of: list[str | None] = [None] * num_pages
        self._free = deque(range(num_pages))
        self._awaiting: list[tuple[int, object]] = []      # (page, fence)
        self._by_owner: dict[str, list[PageRef]] = {}
        self._lock = threading.Lock()

    # ---- accounting --------------------------------------------------------
    def bytes(self) -> int:
        tensors = (self.k_pages, self.v_pages, self.k_norms, self.v_norms)
        return sum(t.numel() * t.element_size() for t in tensors if t is not None)

    def bytes_per_token(self) -> int:
        """Resident KV bytes of one token over all layers."""
        return self.bytes() // (self.num_pages * self.page_size)

    def pages_for(self, tokens: int) -> int:
        return -(-tokens // self.page_size)

    def stats(self) -> dict:
        with self._lock:
            return {"free": len(self._free), "pending": len(self._awaiting),
                    "owned": sum(len(r) for r in self._by_owner.values()),
                    "requests": len(self._by_owner), "total": self.num_pages}

    def held(self, owner: str) -> list[PageRef]:
        with self._lock:
            return list(self._by_owner.get(owner, ()))

    # ---- lifecycle ---------------------------------------------------------
    def ensure(self, owner: str, tokens: int) -> list[PageRef]:
        """Grow `owner`'s reservation to cover `tokens` tokens, or raise."""
        with self._lock:
            refs = self._by_owner.setdefault(owner, [])
            missing = self.pages_for(tokens) - len(refs)
            if missing <= 0:
                return list(refs)
            if len(refs) + missing > self.max_pages_per_request:
                raise PoolExhausted(f"{owner} needs {len(refs) + missing} pages > per-request cap "
                                    f"{self.max_pages_per_request}")
            self._collect_finished()
            if missing > len(self._free):
                raise PoolExhausted(f"{owner} needs {missing} more pages, {len(self._free)} free, "
                                    f"{len(self._awaiting)} awaiting fences")
            for _ in range(missing):
                page = self._free.popleft()
                self._owner_of[page] = owner
                refs.append(PageRef(page, self._generation[page]))
            return list(refs)

    def release(self, owner: str, fence=None) -> int:
        """Revoke `owner`'s pages now; they become reusable once `fence` (recorded
        after the last launch that read them; made here if omitted) completes."""
        if fence is None:
            fence = self._make_fence()
        with self._lock:
            refs = self._by_owner.pop(owner, [])
            for ref in refs:
                self._generation[ref.page] += 1
                self._owner_of[ref.page] = None
                self._awaiting.append((ref.page, fence))
            self._collect_finished()
            return len(refs)

    def reclaim(self) -> int:
        with self._lock:
            return self._collect_finished()

    def _event_done(self, fence) -> bool:
        return fence.query()

    def _collect_finished(self) -> int:
        still_waiting, recycled = [], 0
        for page, fence in self._awaiting:
            if self._event_done(fence):
                self._free.append(page)
                recycled += 1
            else:
                still_waiting.append((page, fence))
        self._awaiting = still_waiting
        return recycled

    def validate(self, owner: str, refs) -> None:
        """Raise `StalePage` unless `owner` holds every ref at its generation."""
        with self._lock:
            for ref in refs:
                if self._owner_of[ref.page] != owner or self._generation[ref.page] != ref.generation:
                    raise StalePage(f"{owner} referenced page {ref.page} gen {ref.generation}; "
                                    f"current owner {self._owner_of[ref.page]!r} "
                                    f"gen {self._generation[ref.page]}")
