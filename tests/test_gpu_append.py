"""GPU parity of packing, quantization and the fused append against the golden
vectors (bytes produced by the reference) and the CPU oracle.  Bit-exact."""
import numpy as np
import pytest
import torch

import cases
from helpers import digest
from oracle import tq_oracle as orc
from winnow_b200 import _lib, packed_attention as pa, packed_backend as pb, workloads
from winnow_b200.cache import _get_quantizer
from winnow_b200.packing import SUPPORTED, pack, unpack
from winnow_b200.page_pool import PagePool

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("bw", SUPPORTED)
def test_pack_unpack_golden(golden, bw):
    g = golden("packing")
    idx = torch.from_numpy(g[f"idx_b{bw}"]).to(DEV)
    packed = pack(idx, bw)
    assert np.array_equal(packed.cpu().numpy(), g[f"packed_b{bw}"])
    assert torch.equal(unpack(packed, bw, 128), idx)


@pytest.mark.parametrize("bw", SUPPORTED)
def test_pack_roundtrip_random(bw):
    g = torch.Generator().manual_seed(bw)
    idx = torch.randint(0, 2 ** bw, (7, 4, 33, 128), generator=g, dtype=torch.uint8)
    packed = pack(idx.to(DEV), bw)
    assert torch.equal(packed.cpu(), orc.pack(idx, bw))
    assert torch.equal(unpack(packed, bw, 128).cpu(), idx)


@pytest.mark.parametrize("c", cases.QUANT_CASES, ids=lambda c: c.name)
def test_quantize_bit_exact(golden, c):
    g = golden("quantize")
    x = cases.quant_input(c)
    tq = _get_quantizer(c.bw, c.D, DEV, 42)
    idx, norms = tq.quantize(x.to(DEV))
    assert idx.shape == x.shape and norms.shape == x.shape[:-1]
    assert np.array_equal(pack(idx, c.bw).cpu().numpy(), g[f"{c.name}/packed"])
    assert np.array_equal(norms.cpu().numpy(), g[f"{c.name}/norms"])
    fused, norms2 = tq.quantize(x.to(DEV), packed=True)
    assert np.array_equal(fused.cpu().numpy(), g[f"{c.name}/packed"])
    assert torch.equal(norms2, norms)


def test_quantize_strided_input():
    tq = _get_quantizer(4, 128, DEV, 42)
    g = torch.Generator().manual_seed(3)
    wide = torch.randn(40, 256, generator=g)
    x = wide[:, :128]
    idx, n = tq.quantize(x.to(DEV)[:, :128])
    ridx, rn = orc.OracleQuantizer.get(4, 128, 42).quantize(x)
    assert torch.equal(idx.cpu(), ridx) and torch.equal(n.cpu(), rn)


def test_quantize_large_matches_oracle():
    """262144 coordinates x 64 at the benchmark's value distribution."""
    w = workloads.WORKLOADS["config2"]
    k, _ = workloads.dense_kv(w, 3)
    x = k[:2, :1024]
    for bw in (4, 6):
        idx, n = _get_quantizer(bw, 128, DEV, 42).quantize(x.to(DEV))
        ridx, rn = orc.OracleQuantizer.get(bw, 128, 42).quantize(x)
        assert int((idx.cpu() != ridx).sum()) == 0
        assert torch.equal(n.cpu(), rn)


@pytest.mark.parametrize("c", cases.APPEND_CASES, ids=lambda c: c.name)
def test_append_bit_exact(golden, c):
    """PagedPackedCache.update through the pool, against the reference's pool
    bytes for the same reservations and inputs."""
    g = golden("append")
    P = cases.append_pool_pages(c)
    pool = PagePool(num_layers=c.layers, num_pages=P, num_kv_heads=c.Hkv, page_size=c.S,
                    nb_k=c.D * c.bw_k // 8, nb_v=c.D * c.bw_v // 8, device=DEV)
    owners = [f"r{b}" for b in range(c.B)]
    for rounds in range(max(-(-(L + c.n) // c.S) for L in c.lengths)):
        for o, L in zip(reversed(owners), reversed(c.lengths)):
            pool.ensure(o, min((rounds + 1) * c.S, L + c.n))
    kq, vq = _get_quantizer(c.bw_k, c.D, DEV, 42), _get_quantizer(c.bw_v, c.D, DEV, 43)
    cache = pb.PagedPackedCache(pool, owners, list(c.lengths), k_quant=kq, v_quant=vq, head_dim=c.D)
    for layer in range(c.layers):
        k, v = cases.append_input(c, layer)
        handle, _ = cache.update(k.to(DEV), v.to(DEV), layer)
        assert isinstance(handle, pa.PackedKV)
    assert np.array_equal(cache._table.cpu().numpy(), g[f"{c.name}/page_table"])
    assert np.array_equal(cache._seq.cpu().numpy(), g[f"{c.name}/seq_lens"])
    assert cache.lengths == [L + c.n for L in c.lengths]
    assert int(cache.status.item()) == 0
    for name in ("k_pages", "v_pages"):
        assert np.array_equal(getattr(pool, name).cpu().numpy(), g[f"{c.name}/{name}"]), name
    for name in ("k_norms", "v_norms"):
        assert np.array_equal(getattr(pool, name).cpu().view(torch.int16).numpy(),
                              g[f"{c.name}/{name}"].view(np.int16)), name


def test_append_refuses_pages_outside_the_pool():
    c = cases.APPEND_CASES[0]
    kq, vq = _get_quantizer(4, 128, DEV, 42), _get_quantizer(4, 128, DEV, 43)
    P = 4
    kp = torch.zeros(P, 2, 16, 64, dtype=torch.uint8, device=DEV)
    vp = torch.zeros_like(kp)
    kn = torch.zeros(P, 2, 16, dtype=torch.float16, device=DEV)
    vn = torch.zeros_like(kn)
    table = torch.tensor([[0, 1], [7, -1], [2, 3]], dtype=torch.int32, device=DEV)   # 7 >= P
    seq = torch.tensor([1, 1, 40], dtype=torch.int32, device=DEV)                    # 40 > 2 pages
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    k, v = cases.append_input(c, 0)
    pb.append_tokens(k.to(DEV), v.to(DEV), kp, kn, vp, vn, table, seq, kq, vq, status=status)
    assert int(status.item()) == (_lib.STATUS_BAD_PAGE | _lib.STATUS_BAD_POSITION)
    assert int(kp[0].count_nonzero()) > 0 and int(kp[1:].count_nonzero()) == 0


def test_config1_cache_bit_exact(golden):
    """Benchmark configuration 1: the whole packed cache built on the GPU equals the
    reference's bytes."""
    g = golden("config1")
    w = workloads.WORKLOADS["config1"]
    k, v = workloads.dense_kv(w, 0)
    kq, vq = _get_quantizer(4, 128, DEV, 42), _get_quantizer(4, 128, DEV, 43)
    kv = pa.pages_from_dense(k[None].to(DEV), v[None].to(DEV), w.seq_lens(), kq, vq, w.page_size,
                             generator=torch.Generator().manual_seed(w.seed))
    assert np.array_equal(kv.page_table.cpu().numpy(), g["page_table"])
    for name in ("k_pages", "v_pages"):
        assert np.array_equal(getattr(kv, name).cpu().numpy(), g[name]), name
    for name in ("k_norms", "v_norms"):
        assert np.array_equal(getattr(kv, name).cpu().view(torch.int16).numpy(),
                              g[name].view(np.int16)), name


@pytest.mark.parametrize("c", [c for c in cases.ATTENTION_CASES if sum(c.lens) * c.Hkv <= 6000],
                         ids=lambda c: c.name)
def test_fixture_builder_matches_reference_pages(golden, c):
    g = golden("attention")
    k, v, q, gen = cases.attention_inputs(c)
    kq, vq = _get_quantizer(c.bw_k, c.D, DEV, 42), _get_quantizer(c.bw_v, c.D, DEV, 43)
    kv = pa.pages_from_dense(k.to(DEV), v.to(DEV), c.lens, kq, vq, c.S, generator=gen)
    for name in ("k_pages", "k_norms", "v_pages", "v_norms", "page_table"):
        assert digest(getattr(kv, name)) == str(g[f"{c.name}/{name}_sha"]), name
