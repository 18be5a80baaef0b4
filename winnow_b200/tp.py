"""KV-head tensor parallelism for the packed decode step.

Every query head reads exactly one kv head (h -> h // n_rep), so kv heads are
independent: rank r of G owns kv heads [r*Hkv/G, (r+1)*Hkv/G) with their query
heads [r*Hq/G, (r+1)*Hq/G), holds only those heads' pages (its pool is
(layers, P, Hkv/G, S, NB)), appends and scans locally, and the step ends with
one all-gather of the (B, Hq/G, 1, D) outputs along the head axis.  The page
table, lengths, rotations and codebooks are replicated.  No rank ever reads
another rank's pages.  The reference has no multi-GPU form of this path; the
partition follows its head mapping (turboquant_kv/packed_attention.py:168-170).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def head_shard(rank: int, world: int, q_heads: int, kv_heads: int) -> tuple[slice, slice]:
    """(query-head slice, kv-head slice) owned by `rank`."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside a world of {world}")
    if q_heads % kv_heads:
        raise ValueError(f"Hq={q_heads} is not a multiple of Hkv={kv_heads}")
    if kv_heads % world:
        raise ValueError(f"{kv_heads} kv heads do not shard over {world} ranks; "
                         "run replicas instead")
    hkv, hq = kv_heads // world, q_heads // world
    return slice(rank * hq, (rank + 1) * hq), slice(rank * hkv, (rank + 1) * hkv)


class HeadGather:
    """All-gather of per-rank (B, Hq/G, 1, D) outputs into (B, Hq, 1, D).

    `local` is the buffer the rank's decode call writes (a view of the gather
    buffer, so the collective needs no staging copy); `gather()` runs the
    collective on the current stream and returns the assembled tensor.
    """

    def __init__(self, batch: int, q_heads: int, head_dim: int, dtype, device, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if q_heads % self.world:
            raise ValueError(f"{q_heads} query heads do not shard over {self.world} ranks")
        self.hq = q_heads // self.world
        self._parts = torch.zeros(self.world, batch, self.hq, 1, head_dim, dtype=dtype, device=device)
        self.full = torch.zeros(batch, q_heads, 1, head_dim, dtype=dtype, device=device)

    @property
    def local(self) -> torch.Tensor:
        return self._parts[self.rank] if self.world > 1 else self.full

    def gather(self) -> torch.Tensor:
        if self.world == 1:
            return self.full
        flat = self._parts.view(self.world, -1)
        if flat.is_cuda:
            dist.all_gather_into_tensor(self._parts.view(-1), flat[self.rank], group=self.group)
        else:                                    # gloo: list form
            parts = [flat[r] for r in range(self.world)]
            dist.all_gather(parts, flat[self.rank].clone(), group=self.group)
        B = self.full.shape[0]
        self.full.view(B, self.world, self.hq, 1, -1).copy_(self._parts.permute(1, 0, 2, 3, 4))
        return self.full


class PeerExchange:
    """Output exchange fused into the decode call: no collective library call.

    Every rank allocates the same symmetric buffer (two full (B, Hq, 1, D)
    outputs, used alternately, and a flag array) and maps its peers' copies.
    The merge kernel of `wtq_decode_exchange` stores this rank's head rows into
    every rank's buffer over NVLink and publishes the step number; a one-block
    kernel (`wtq_exchange_wait`) then waits, with a bounded number of polls,
    until all ranks have published.  Plain peer stores only, no multicast.
    """

    SPIN_LIMIT = 4_000_000            # polls of ~100 ns: gives up after a fraction of a second

    def __init__(self, batch: int, q_heads: int, head_dim: int, dtype, device, group=None,
                 spin_limit: int | None = None):
        """`spin_limit`: polls of a peer's flag before the wait gives up (default
        SPIN_LIMIT); size it to the rank skew the serving loop expects.  After a
        timeout the buffer still holds the late rank's previous rows: the result
        of a step is valid only while `status` is zero (`check()`)."""
        import torch.distributed._symmetric_memory as symm_mem
        self.spin_limit = int(spin_limit) if spin_limit else self.SPIN_LIMIT
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if q_heads % self.world:
            raise ValueError(f"{q_heads} query heads do not shard over {self.world} ranks")
        self.hq = q_heads // self.world
        el = torch.empty((), dtype=dtype).element_size()
        self.out_elems = batch * q_heads * head_dim
        out_bytes = -(-self.out_elems * el // 256) * 256
        total = 2 * out_bytes + 256
        self._buf = symm_mem.empty(total, dtype=torch.uint8, device=device)
        self._buf.zero_()
        self._hdl = symm_mem.rendezvous(self._buf, self.group)
        bases = [int(p) for p in self._hdl.buffer_ptrs]
        dev = torch.device(device)
        self._peer_out = [torch.tensor([b + i * out_bytes for b in bases], dtype=torch.int64, device=dev)
                          for i in range(2)]
        self._peer_flags = torch.tensor([b + 2 * out_bytes for b in bases], dtype=torch.int64, device=dev)
        self.full = [self._buf[i * out_bytes: i * out_bytes + self.out_elems * el].view(dtype)
                     .view(batch, q_heads, 1, head_dim) for i in range(2)]
        self.flags = self._buf[2 * out_bytes: 2 * out_bytes + 4 * self.world].view(torch.int32)
        self.done = torch.zeros(1, dtype=torch.int32, device=dev)
        self.step_dev = torch.zeros(4, dtype=torch.int32, device=dev)   # calls, waits, blocks per call
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.step = 0
        self.device = dev
        torch.cuda.synchronize(dev)
        dist.barrier(self.group)          # every rank's flags are zero before anyone publishes

    def descriptor(self):
        """The wtq_exchange_t of this rank (constant: the step number lives in
        device memory and is advanced by the kernels)."""
        from . import _lib
        if not hasattr(self, "_desc"):
            ex = _lib.Exchange()
            ex.peer_out[0] = self._peer_out[0].data_ptr()
            ex.peer_out[1] = self._peer_out[1].data_ptr()
            ex.peer_flags = self._peer_flags.data_ptr()
            ex.out_strides[0], ex.out_strides[1] = self.full[0].stride(0), self.full[0].stride(1)
            ex.rank, ex.world, ex.head_offset = self.rank, self.world, self.rank * self.hq
            ex.step_counter = self.step_dev.data_ptr()
            ex.done_counter = self.done.data_ptr()
            self._desc = ex
            self._wait = _lib.lib().wtq_exchange_wait
            self._wait_args = (self.flags.data_ptr(), self.world, self.step_dev.data_ptr(),
                               self.spin_limit, self.status.data_ptr())
        return self._desc

    def wait(self) -> None:
        """Enqueue the bounded wait for every rank's rows of the latest call."""
        rc = self._wait(*self._wait_args, torch.cuda.current_stream(self.device).cuda_stream)
        if rc:
            from . import _lib
            _lib.check(rc)

    def result(self, call_number: int) -> torch.Tensor:
        """Full output of call number `call_number` (1, 2, ...), valid once the
        wait enqueued after that call has run."""
        return self.full[call_number & 1]

    def timed_out(self) -> bool:
        """Host check of the status word (synchronises)."""
        from . import _lib
        return bool(int(self.status.item()) & _lib.STATUS_EXCHANGE_TIMEOUT)

    def check(self) -> None:
        """Raise if any wait since the last check gave up (synchronises with
        the device: call it where the caller syncs anyway, e.g. before sampling).
        The status word is cleared so that later steps are assessed on their own."""
        from . import _lib
        word = int(self.status.item())
        if word:
            self.status.zero_()
            raise _lib.BackendError(
                f"output exchange: status {word:#x} after step {self.step} (bit "
                f"{_lib.STATUS_EXCHANGE_TIMEOUT}: a peer's rows did not arrive within "
                f"{self.spin_limit} polls; the gathered buffer holds stale rows for it)")


class TensorParallelDecode:
    """One rank's side of the sharded decode step.

    `kv` is this rank's `PackedKV` (its kv heads only) and `q_local` its
    (B, Hq/G, 1, D) query heads.  `step()` scans the local pages into this
    rank's slot of the gather buffer and returns the full (B, Hq, 1, D) output
    after the all-gather.
    """

    def __init__(self, q_local: torch.Tensor, kv, scale: float, q_heads: int, *, group=None,
                 num_splits: int | None = None, check_page_ids: bool = True,
                 exchange: str = "nccl", spin_limit: int | None = None):
        """`exchange="nccl"`: scan, then `all_gather_into_tensor` and a permuting
        copy.  `exchange="peer"`: the merge kernel writes every rank's buffer
        itself (`PeerExchange`); shapes without a tensor-core kernel fall back to
        "nccl" (see `self.exchange`).  The choice is agreed on by all ranks: the
        peer form is used only if every rank could set it up, so no rank ends up
        in a collective the others never enter."""
        from .packed_attention_cuda import DecodePlan
        B, hq, _, D = q_local.shape
        self.exchange = exchange
        self.peer = None
        if exchange == "peer":
            why = ""
            try:
                # (symmetric-memory set-up is itself collective: every rank enters it)
                self.peer = PeerExchange(B, q_heads, D, q_local.dtype, q_local.device, group,
                                         spin_limit=spin_limit)
            except _lib_error() as exc:
                self.peer, why = None, f"{type(exc).__name__}: {exc}"
            if self.peer is not None:
                try:
                    if hq != self.peer.hq:
                        raise ValueError(f"expected {self.peer.hq} local query heads, got {hq}")
                    self.plan = DecodePlan(q_local, kv, scale, num_splits=num_splits,
                                           out=self.peer.full[0][:, :hq],
                                           check_page_ids=check_page_ids)
                    self.plan.run_exchange(self.peer.descriptor(), dry_run=True)
                except _lib_error() as exc:
                    why = f"{type(exc).__name__}: {exc}"
            if not _all_ranks_agree(why == "", q_local.device, group):
                self.peer = None
                self.exchange = f"nccl (peer exchange unavailable on some rank{': ' + why if why else ''})"
        if self.peer is None:
            self.heads = HeadGather(B, q_heads, D, q_local.dtype, q_local.device, group)
            if hq != self.heads.hq:
                raise ValueError(f"expected {self.heads.hq} local query heads, got {hq}")
            self.plan = DecodePlan(q_local, kv, scale, num_splits=num_splits, out=self.heads.local,
                                   check_page_ids=check_page_ids)

    def step(self, check: bool = False) -> torch.Tensor:
        """One decode step; returns the full (B, Hq, 1, D) output.  On the peer
        path the wait for the other ranks' rows is bounded: if a rank is later
        than `spin_limit` polls the wait gives up, sets the status word and the
        returned buffer still holds that rank's previous rows.  The output is
        therefore valid only while the status is zero: pass `check=True` (one
        device synchronisation per step) or call `check()` at the next point
        where the caller synchronises anyway; both raise `BackendError`."""
        if self.peer is None:
            self.plan.run()
            return self.heads.gather()
        self.peer.step += 1
        self.plan.run_exchange(self.peer.descriptor())
        self.peer.wait()
        if check:
            self.peer.check()
        return self.peer.result(self.peer.step)

    def check(self) -> None:
        """Raise `BackendError` if a bounded wait gave up since the last check."""
        if self.peer is not None:
            self.peer.check()


def _all_ranks_agree(ok: bool, device, group) -> bool:
    """True when `ok` holds on every rank of the group (one small all-reduce)."""
    if not dist.is_initialized():
        return ok
    dev = device if dist.get_backend(group) == "nccl" else "cpu"
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    return bool(int(flag.item()))


def _lib_error():
    from . import _lib
    return (_lib.BackendError, RuntimeError, AttributeError, ImportError)
