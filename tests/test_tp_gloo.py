"""KV-head sharding over two gloo ranks on the CPU: each rank owns half of the
kv heads with their query heads, computes attention over its shard alone (the
oracle stands in for the CUDA kernel here), and the head all-gather must
reassemble exactly the unsharded result."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import cases
from helpers import oracle_case
from oracle import tq_oracle as orc
from winnow_b200 import tp


def test_head_shard_math():
    assert tp.head_shard(0, 1, 32, 8) == (slice(0, 32), slice(0, 8))
    assert tp.head_shard(3, 8, 64, 8) == (slice(24, 32), slice(3, 4))
    assert tp.head_shard(1, 2, 8, 2) == (slice(4, 8), slice(1, 2))
    with pytest.raises(ValueError):
        tp.head_shard(0, 4, 8, 2)           # 2 kv heads cannot shard over 4 ranks
    with pytest.raises(ValueError):
        tp.head_shard(2, 2, 8, 2)
    # every query head lands on the rank that owns its kv head
    for world in (1, 2, 4, 8):
        for h in range(64):
            owner = [r for r in range(world) if h in range(64)[tp.head_shard(r, world, 64, 8)[0]]]
            kv_owner = [r for r in range(world) if (h // 8) in range(8)[tp.head_shard(r, world, 64, 8)[1]]]
            assert owner == kv_owner and len(owner) == 1


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, case_index, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        c = cases.ATTENTION_CASES[case_index]
        q, kv, _ = oracle_case(c)
        scale = orc.default_scale(c.D)
        full = orc.tiled_attention(q, kv, scale)
        qs, ks = tp.head_shard(rank, world, c.Hq, c.Hkv)
        shard = orc.OracleKV(**{**kv.__dict__,
                                "k_pages": kv.k_pages[:, ks].contiguous(),
                                "k_norms": kv.k_norms[:, ks].contiguous(),
                                "v_pages": kv.v_pages[:, ks].contiguous(),
                                "v_norms": kv.v_norms[:, ks].contiguous()})
        heads = tp.HeadGather(c.B, c.Hq, c.D, torch.float32, "cpu")
        assert heads.local.shape == (c.B, c.Hq // world, 1, c.D)
        heads.local.copy_(orc.tiled_attention(q[:, qs], shard, scale))
        got = heads.gather()
        results[rank] = float((got - full).abs().max())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("case_index", [3, 5])        # gqa8_2 (Hkv 2), four_bit (Hkv 4)
def test_two_ranks_reassemble_the_unsharded_output(case_index):
    world = 2
    port = _free_port()
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(world, port, case_index, results), nprocs=world, join=True)
        assert sorted(results.keys()) == [0, 1]
        assert all(err < 1e-6 for err in results.values()), dict(results)
