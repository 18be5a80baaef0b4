"""KV-head tensor parallelism on real GPUs: two ranks, one per GPU, each with
half of the kv heads' pages; after the all-gather every rank must hold the
unsharded output.  Skipped on a box with a single GPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import cases

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, name, results):
    from helpers import oracle_case, to_device
    from oracle import tq_oracle as orc
    from winnow_b200 import packed_attention as pa, tp
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    try:
        c = next(x for x in cases.ATTENTION_CASES if x.name == name)
        q, okv, _ = oracle_case(c)
        scale = orc.default_scale(c.D)
        full = orc.tiled_attention(q, okv, scale)
        dev = torch.device("cuda", rank)
        qs, ks = tp.head_shard(rank, world, c.Hq, c.Hkv)
        kv = to_device(okv, dev)
        shard = pa.PackedKV(kv.k_pages[:, ks].contiguous(), kv.k_norms[:, ks].contiguous(),
                            kv.v_pages[:, ks].contiguous(), kv.v_norms[:, ks].contiguous(),
                            kv.page_table, kv.seq_lens, kv.k_quant, kv.v_quant, kv.head_dim)
        errs = []
        for exchange in ("nccl", "peer"):
            q_local = q[:, qs].contiguous().to(dev)
            runner = tp.TensorParallelDecode(q_local, shard, scale, c.Hq, exchange=exchange)
            out = runner.step()
            errs.append(float((out.float().cpu() - full).abs().max()))
            # buffers are reused step after step; the query changes in place
            for i in range(1, 6):
                qi = q * (1.0 + 0.25 * i)
                q_local.copy_(qi[:, qs])
                out = runner.step()
                ref = orc.tiled_attention(qi, okv, scale)
                errs.append(float((out.float().cpu() - ref).abs().max()))
            torch.cuda.synchronize()
            if runner.peer is not None:
                assert not runner.peer.timed_out()
            elif exchange == "peer":
                errs.append(("fallback", runner.exchange))
        results[rank] = errs
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("name", ["val_long", "six_bit"])
def test_two_gpus_kv_head_sharding(name):
    world, port = 2, _free_port()
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(world, port, name, results), nprocs=world, join=True)
        assert sorted(results.keys()) == [0, 1]
        for errs in results.values():
            numeric = [e for e in errs if not isinstance(e, tuple)]
            assert max(numeric) <= 2e-3, dict(results)
        if name == "val_long":                      # a tensor-core shape: the fused exchange must run
            assert not any(isinstance(e, tuple) for errs in results.values() for e in errs), dict(results)
