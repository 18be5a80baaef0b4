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


class TensorParallelDecode:
    """One rank's side of the sharded decode step.

    `kv` is this rank's `PackedKV` (its kv heads only) and `q_local` its
    (B, Hq/G, 1, D) query heads.  `step()` scans the local pages into this
    rank's slot of the gather buffer and returns the full (B, Hq, 1, D) output
    after the all-gather.
    """

    def __init__(self, q_local: torch.Tensor, kv, scale: float, q_heads: int, *, group=None,
                 num_splits: int | None = None, check_page_ids: bool = True):
        from .packed_attention_cuda import DecodePlan
        B, hq, _, D = q_local.shape
        self.heads = HeadGather(B, q_heads, D, q_local.dtype, q_local.device, group)
        if hq != self.heads.hq:
            raise ValueError(f"expected {self.heads.hq} local query heads, got {hq}")
        self.plan = DecodePlan(q_local, kv, scale, num_splits=num_splits, out=self.heads.local,
                               check_page_ids=check_page_ids)

    def step(self) -> torch.Tensor:
        self.plan.run()
        return self.heads.gather()
