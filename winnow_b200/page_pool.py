"""Page pool for packed KV: request-scoped reservations, fenced reuse, and a
page table that lives on the device.

Public behaviour follows the reference allocator
(turboquant_kv/page_pool.py:62-175): page id p means page p of every layer, a
page is held under (owner, generation), `release` revokes at once but the page
only becomes reusable when the fence recorded after the last launch that could
read it has completed, and admission is all-or-nothing (`ensure` raises
`PoolExhausted`, never evicts).  The tensors it owns are what the CUDA kernels
read and write:

    k_pages, v_pages  (layers, P, Hkv, S, NB) uint8   packed codes
    k_norms, v_norms  (layers, P, Hkv, S)     fp16

The bookkeeping is built for a serving loop that runs the same batch step after
step: page state is held in flat arrays (generation, owner slot), a reservation
remembers its pages in order, pages retired by one `release` share one fence
record, a whole batch can be grown in one all-or-nothing call (`ensure_many`),
and `DeviceTable` keeps the batch's (B, width) int32 page table in device
memory, rewriting only the rows whose reservation changed since the last
forward instead of rebuilding and copying the table every time.
"""
from __future__ import annotations

import threading
from dataclasses import dataclass

import numpy as np
import torch


class PoolExhausted(RuntimeError):
    """Not enough free pages; refuse or queue the request."""


class StalePage(RuntimeError):
    """A launch referenced a page its caller no longer owns."""


@dataclass(frozen=True)
class PageRef:
    page: int
    generation: int


class _Finished:
    """Fence of work that has nothing outstanding (CPU bookkeeping only)."""

    def query(self) -> bool:
        return True

    def synchronize(self) -> None:
        return None


def default_fence(device: torch.device):
    """An event recorded now on the device's current stream."""
    if torch.device(device).type != "cuda":
        return _Finished()
    event = torch.cuda.Event()
    event.record(torch.cuda.current_stream(device))
    return event


class _Reservation:
    """Pages one owner holds, in token order, with the generation each was taken at."""

    __slots__ = ("slot", "pages", "generations", "version")

    def __init__(self, slot: int):
        self.slot = slot
        self.pages: list[int] = []
        self.generations: list[int] = []
        self.version = 0                      # bumped whenever `pages` changes

    def refs(self) -> list[PageRef]:
        return [PageRef(p, g) for p, g in zip(self.pages, self.generations)]


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
        self._new_fence = fence_factory or (lambda: default_fence(self.device))
        # page state: generation counter and the slot of the reservation holding it (-1: none)
        self._gen = np.zeros(num_pages, dtype=np.int64)
        self._slot_of = np.full(num_pages, -1, dtype=np.int64)
        self._free: list[int] = list(range(num_pages - 1, -1, -1))     # stack; page 0 on top
        self._retired: list[tuple[object, list[int]]] = []             # (fence, pages) per release
        self._held: dict[str, _Reservation] = {}
        self._next_slot = 0
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
            return {"free": len(self._free),
                    "pending": sum(len(pages) for _, pages in self._retired),
                    "owned": sum(len(r.pages) for r in self._held.values()),
                    "requests": len(self._held), "total": self.num_pages}

    def held(self, owner: str) -> list[PageRef]:
        with self._lock:
            res = self._held.get(owner)
            return res.refs() if res is not None else []

    # ---- lifecycle ---------------------------------------------------------
    def _grow(self, owner: str, res: _Reservation, missing: int) -> None:
        for _ in range(missing):
            page = self._free.pop()
            self._slot_of[page] = res.slot
            res.pages.append(page)
            res.generations.append(int(self._gen[page]))
        res.version += 1

    def _reservation(self, owner: str) -> _Reservation:
        res = self._held.get(owner)
        if res is None:
            res = self._held[owner] = _Reservation(self._next_slot)
            self._next_slot += 1
        return res

    def ensure(self, owner: str, tokens: int) -> list[PageRef]:
        """Grow `owner`'s reservation to cover `tokens` tokens, or raise."""
        with self._lock:
            res = self._reservation(owner)
            missing = self.pages_for(tokens) - len(res.pages)
            if missing > 0:
                if len(res.pages) + missing > self.max_pages_per_request:
                    raise PoolExhausted(f"request {owner!r} would hold {len(res.pages) + missing} pages; "
                                        f"the per-request limit is {self.max_pages_per_request}")
                self._sweep()
                if missing > len(self._free):
                    waiting = sum(len(pages) for _, pages in self._retired)
                    raise PoolExhausted(f"request {owner!r} is {missing} pages short: {len(self._free)} "
                                        f"free, {waiting} still behind a fence")
                self._grow(owner, res, missing)
            return res.refs()

    def ensure_many(self, owners, tokens) -> None:
        """Grow every (owner, tokens) pair of a batch, or none of them: the
        whole step's demand is checked against the free list first."""
        with self._lock:
            demand = []
            for owner, want in zip(owners, tokens):
                res = self._reservation(owner)
                missing = max(0, self.pages_for(want) - len(res.pages))
                if len(res.pages) + missing > self.max_pages_per_request:
                    raise PoolExhausted(f"request {owner!r} would hold {len(res.pages) + missing} pages; "
                                        f"the per-request limit is {self.max_pages_per_request}")
                demand.append((owner, res, missing))
            total = sum(m for _, _, m in demand)
            if total:
                self._sweep()
                if total > len(self._free):
                    raise PoolExhausted(f"the batch is {total} pages short: {len(self._free)} free")
                for owner, res, missing in demand:
                    if missing:
                        self._grow(owner, res, missing)

    def release(self, owner: str, fence=None) -> int:
        """Revoke `owner`'s pages now; they become reusable once `fence` (recorded
        after the last launch that read them; made here if omitted) completes."""
        if fence is None:
            fence = self._new_fence()
        with self._lock:
            res = self._held.pop(owner, None)
            if res is None or not res.pages:
                self._sweep()
                return 0
            pages = np.asarray(res.pages, dtype=np.int64)
            self._gen[pages] += 1                 # every outstanding PageRef is stale from here on
            self._slot_of[pages] = -1
            self._retired.append((fence, res.pages))
            self._sweep()
            return len(res.pages)

    def reclaim(self) -> int:
        with self._lock:
            return self._sweep()

    def _sweep(self) -> int:
        """Move the pages of every finished fence back to the free stack."""
        if not self._retired:
            return 0
        recycled, waiting = 0, []
        for fence, pages in self._retired:
            if fence.query():
                self._free.extend(reversed(pages))
                recycled += len(pages)
            else:
                waiting.append((fence, pages))
        self._retired = waiting
        return recycled

    def validate(self, owner: str, refs) -> None:
        """Raise `StalePage` unless `owner` holds every ref at its generation."""
        with self._lock:
            res = self._held.get(owner)
            slot = res.slot if res is not None else -2
            for ref in refs:
                if self._slot_of[ref.page] != slot or self._gen[ref.page] != ref.generation:
                    raise StalePage(f"request {owner!r} used page {ref.page} taken at generation "
                                    f"{ref.generation}; the page is now at generation "
                                    f"{int(self._gen[ref.page])} and "
                                    f"{'unowned' if self._slot_of[ref.page] < 0 else 'held by another request'}")

    def _snapshot(self, owner: str):
        """(version, pages) of `owner`'s reservation, validated as a whole."""
        with self._lock:
            res = self._held.get(owner)
            if res is None:
                return -1, []
            pages = np.asarray(res.pages, dtype=np.int64)
            if len(pages) and (np.any(self._slot_of[pages] != res.slot)
                               or np.any(self._gen[pages] != np.asarray(res.generations))):
                raise StalePage(f"request {owner!r} holds a page that was released")
            return res.version, list(res.pages)


class DeviceTable:
    """The (B, width) int32 page table of a fixed batch of owners, kept in device
    memory across forwards.  `refresh(needed_tokens)` re-reads only the
    reservations whose version changed and writes those rows (one small
    host-to-device copy per changed row, none in the common decode step where
    no sequence crossed a page boundary); unused entries are -1.  The tensor
    object never changes, so launches marshalled against it (and CUDA graphs)
    stay valid."""

    def __init__(self, pool: PagePool, owners, width: int, device=None):
        self.pool, self.owners, self.width = pool, list(owners), int(width)
        dev = torch.device(device) if device is not None else pool.device
        self.table = torch.full((len(self.owners), self.width), -1, dtype=torch.int32, device=dev)
        self._seen = [None] * len(self.owners)
        self._stage = torch.empty(self.width, dtype=torch.int32,
                                  pin_memory=dev.type == "cuda")

    def refresh(self, needed_tokens=None) -> int:
        """Bring the device table up to date; returns the rows rewritten.
        `needed_tokens[b]`: tokens sequence b must be able to hold (checked
        against its reservation, `StalePage` if short)."""
        changed = 0
        for b, owner in enumerate(self.owners):
            version, pages = self.pool._snapshot(owner)
            if needed_tokens is not None and self.pool.pages_for(needed_tokens[b]) > len(pages):
                raise StalePage(f"request {owner!r} holds {len(pages)} pages, the step needs "
                                f"{self.pool.pages_for(needed_tokens[b])}")
            if self._seen[b] == (version, len(pages)):
                continue
            if len(pages) > self.width:
                raise PoolExhausted(f"request {owner!r} holds {len(pages)} pages; this table is "
                                    f"{self.width} wide")
            self._stage.fill_(-1)
            if pages:
                self._stage[:len(pages)] = torch.as_tensor(pages, dtype=torch.int32)
            self.table[b].copy_(self._stage, non_blocking=False)
            self._seen[b] = (version, len(pages))
            changed += 1
        return changed
