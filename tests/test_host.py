"""Host-side logic that needs no GPU: page pool, contract checks, planner,
workload generators, and the refusal to run without CUDA."""
import pytest
import torch

import cases
from helpers import oracle_case, to_device
from winnow_b200 import _lib, dispatch, packed_attention as pa, packed_backend as pb, workloads
from winnow_b200.cache import TurboQuantMSE, _get_quantizer
from winnow_b200.packing import SUPPORTED, pack, packed_bytes
from winnow_b200.page_pool import PagePool, PoolExhausted, StalePage


class Pending:
    def __init__(self):
        self.done = False

    def query(self):
        return self.done

    def synchronize(self):
        pass


def pool(**kw):
    args = dict(num_layers=2, num_pages=6, num_kv_heads=2, page_size=4, nb_k=8, nb_v=12)
    args.update(kw)
    return PagePool(**args)


def test_pool_shapes_and_accounting():
    p = pool()
    assert p.k_pages.shape == (2, 6, 2, 4, 8) and p.v_pages.shape == (2, 6, 2, 4, 12)
    assert p.k_norms.shape == (2, 6, 2, 4) and p.k_norms.dtype == torch.float16
    assert p.bytes() == 2 * 6 * 2 * 4 * (8 + 12 + 4)
    assert p.bytes_per_token() == 2 * 2 * (8 + 12 + 4)
    assert p.pages_for(0) == 0 and p.pages_for(4) == 1 and p.pages_for(5) == 2


def test_pool_allocation_is_all_or_nothing():
    p = pool(max_pages_per_request=3)
    assert len(p.ensure("a", 9)) == 3
    with pytest.raises(PoolExhausted):
        p.ensure("a", 13)                       # per-request cap
    p.ensure("b", 8)
    with pytest.raises(PoolExhausted):
        p.ensure("c", 8)                        # only one page left
    assert p.stats() == {"free": 1, "pending": 0, "owned": 5, "requests": 3, "total": 6}


def test_release_bumps_generation_and_waits_for_the_fence():
    fence = Pending()
    p = pool()
    refs = p.ensure("a", 8)
    p.validate("a", refs)
    assert p.release("a", fence) == 2
    with pytest.raises(StalePage):
        p.validate("a", refs)
    assert p.stats()["pending"] == 2 and p.stats()["free"] == 4
    with pytest.raises(PoolExhausted):
        p.ensure("b", 20)                       # pending pages are not reusable
    fence.done = True
    assert p.reclaim() == 2 and p.stats()["free"] == 6
    again = p.ensure("b", 24)
    assert {r.page for r in again} == set(range(6))
    assert any(r.generation == 1 for r in again)


def test_batch_reservation_and_device_table():
    """`ensure_many` grows a whole batch or nothing; `DeviceTable` rewrites only
    the rows whose reservation changed and refuses a step its pages cannot hold."""
    from winnow_b200.page_pool import DeviceTable
    p = pool(num_pages=8)
    p.ensure_many(["a", "b"], [5, 4])                       # 2 + 1 pages
    assert p.stats()["owned"] == 3
    with pytest.raises(PoolExhausted):
        p.ensure_many(["a", "b", "c"], [9, 9, 13])           # 1 + 2 + 4 more > 5 free
    assert p.stats()["owned"] == 3                           # nothing was taken
    t = DeviceTable(p, ["a", "b"], width=4, device="cpu")
    assert t.refresh([5, 4]) == 2
    assert t.table.tolist() == [[0, 1, -1, -1], [2, -1, -1, -1]]
    assert t.refresh([6, 4]) == 0                            # nobody crossed a page boundary
    p.ensure_many(["a", "b"], [6, 5])
    assert t.refresh([6, 5]) == 1 and t.table[1].tolist() == [2, 3, -1, -1]
    with pytest.raises(StalePage):
        t.refresh([6, 9])                                    # b holds 2 pages, 9 tokens need 3
    p.release("a", Pending())
    with pytest.raises(StalePage):
        t.refresh([6, 5])                                    # a's pages are gone
    with pytest.raises(PoolExhausted):
        p.ensure_many(["z"], [4 * 9])                        # beyond the per-request limit


def test_contract_rejections_on_metadata():
    c = cases.ATTENTION_CASES[3]
    q, okv, _ = oracle_case(c)
    kv = to_device(okv, "cpu")
    pa.check_contract(q, kv)
    with pytest.raises(pa.UnsupportedLayout):
        pa.check_contract(q[..., :32], kv)
    with pytest.raises(pa.UnsupportedLayout):
        pa.check_contract(q[:, :7], kv)
    with pytest.raises(pa.UnsupportedLayout):
        pa.check_contract(q, pa.PackedKV(**{**kv.__dict__, "page_table": kv.page_table.long()}))
    bad = pa.PackedKV(**{**kv.__dict__, "page_table": kv.page_table.clone()})
    bad.page_table[0, 0] = kv.k_pages.shape[0]
    with pytest.raises(pa.UnsupportedLayout):
        pa.check_contract(q, bad)
    pa.check_contract(q, bad, check_page_ids=False)     # id check is the only host read
    with pytest.raises(pa.UnsupportedLayout):
        pa.check_contract(q, pa.PackedKV(**{**kv.__dict__, "seq_lens": kv.seq_lens + 1000}))
    with pytest.raises(pa.UnsupportedLayout):
        pa.check_contract(q, pa.PackedKV(**{**kv.__dict__, "k_norms": kv.k_norms.float()}))


def test_no_cpu_path():
    """CPU tensors never reach a silent fallback."""
    c = cases.ATTENTION_CASES[3]
    q, okv, _ = oracle_case(c)
    kv = to_device(okv, "cpu")
    from winnow_b200.packed_attention_cuda import packed_decode_attention
    with pytest.raises(pa.UnsupportedLayout):
        packed_decode_attention(q, kv, 1.0)
    with pytest.raises(_lib.BackendError):
        pack(torch.zeros(2, 128, dtype=torch.uint8), 4)
    with pytest.raises(_lib.BackendError):
        TurboQuantMSE(4, 128).quantize(torch.zeros(2, 128))
    with pytest.raises(RuntimeError):
        pb.select_decode_backend(q, kv, "auto")
    with pytest.raises(ValueError):
        pb.select_decode_backend(q, kv, "no_such_backend")


def test_packed_bytes_and_widths():
    assert SUPPORTED == (2, 3, 4, 5, 6, 8)
    assert packed_bytes(128, 3) == 48 and packed_bytes(128, 4) == 64 and packed_bytes(128, 6) == 96
    with pytest.raises(ValueError):
        packed_bytes(9, 3)


def test_quantizer_construction_matches_golden(golden):
    g = golden("codebooks")
    for bw in (4, 6, 8):
        tq = _get_quantizer(bw, 128, "cpu", 42)
        assert (tq.centroids.numpy() == g[f"centroids_d128_b{bw}"]).all()
        assert (tq.boundaries.numpy() == g[f"boundaries_d128_b{bw}"]).all()
    assert (_get_quantizer(4, 128, "cpu", 43).Pi.numpy() == g["pi_d128_s43"]).all()
    assert _get_quantizer(4, 128, "cpu", 42) is _get_quantizer(4, 128, "cpu", 42)


def test_planner_controls():
    d = dispatch.default_dispatcher()
    shape = dispatch.Shape(16, 8, 8192, 128, 4)
    ok = dispatch.NumericalContract.quantization_aware()
    b200 = dispatch.Hardware("NVIDIA B200", (10, 0))
    assert d.select(b200, shape, ok).backend == dispatch.BACKEND
    assert d.select(dispatch.Hardware("NVIDIA RTX A6000", (8, 6)), shape, ok).backend == "none"
    assert d.select(dispatch.Hardware("unknown", None), shape, ok).backend == "none"
    assert d.select(b200, shape, dispatch.NumericalContract.reference_exact()).backend == "none"
    assert d.select(b200, shape, ok, available=()).backend == "none"
    assert d.select(b200, dispatch.Shape(1, 1, 8, 9, 3), ok).backend == "none"


def test_model_gate():
    class Cfg:
        architectures = ["Qwen2ForCausalLM"]
        hidden_size, num_attention_heads, num_key_value_heads, num_hidden_layers = 1024, 8, 2, 3
    pb.check_model(Cfg, 4)
    pb.check_model(Cfg, 4, bit_width_v=6)
    Cfg2 = type("C", (Cfg,), {"architectures": ["GPT2LMHeadModel"]})
    with pytest.raises(pb.UnsupportedModel):
        pb.check_model(Cfg2, 4)
    Cfg3 = type("C", (Cfg,), {"use_sliding_window": True})
    with pytest.raises(pb.UnsupportedModel):
        pb.check_model(Cfg3, 4)
    p = pb.make_pool(Cfg, bit_width=4, bit_width_v=6, num_pages=4, page_size=16, device="cpu")
    assert p.k_pages.shape[-1] == 64 and p.v_pages.shape[-1] == 96


def test_workload_definitions():
    w2 = workloads.WORKLOADS["config2"]
    assert w2.algorithmic_bytes() == 16 * 8192 * 8 * 132 + 4 * 16 * 512 + 16 * 32 * 128 * 4
    w5 = workloads.WORKLOADS["config5"]
    lens = w5.seq_lens()
    assert len(lens) == 128 and min(lens) >= 512 and max(lens) <= 32768 and lens == w5.seq_lens()
    table, total = workloads.page_assignment(workloads.WORKLOADS["config1"])
    assert total == 64 and sorted(table[0].tolist()) == list(range(64))
    k, v = workloads.dense_kv(workloads.WORKLOADS["config1"], 0)
    assert k.shape == (2, 1024, 128)


def test_merge_partials_and_rotations_follow_the_reference_algebra():
    """`merge_partials` combines online-softmax states as the oracle's merge
    does (empty states carry -inf and weigh nothing); `rotate_query` /
    `rotate_output` are q Pi^T and a Pi."""
    import torch
    from oracle import tq_oracle as orc
    from winnow_b200 import packed_attention as pa
    g = torch.Generator().manual_seed(5)
    m1, m2 = torch.randn(2, 3, 1, generator=g), torch.randn(2, 3, 1, generator=g)
    m2[0, 0, 0] = float("-inf")
    l1, l2 = torch.rand(2, 3, 1, generator=g) + 0.1, torch.rand(2, 3, 1, generator=g)
    l2[0, 0, 0] = 0.0
    a1, a2 = torch.randn(2, 3, 1, 8, generator=g), torch.randn(2, 3, 1, 8, generator=g)
    a2[0, 0, 0] = 0.0
    got = pa.merge_partials((m1, l1, a1), (m2, l2, a2))
    ref = orc.merge_states((m1, l1, a1), (m2, l2, a2))
    for x, y in zip(got, ref):
        assert torch.equal(x, y)
    both_empty = pa.merge_partials((m2[:1, :1], l2[:1, :1], a2[:1, :1]), (m2[:1, :1], l2[:1, :1], a2[:1, :1]))
    assert float(both_empty[1].abs().max()) == 0.0 and not torch.isnan(both_empty[2]).any()
    Pi = orc.rotation_matrix(8, 7)
    x = torch.randn(4, 8, generator=g)
    assert torch.equal(pa.rotate_query(x, Pi), x @ Pi.T)
    assert torch.equal(pa.rotate_output(x, Pi), x @ Pi)
    assert torch.allclose(pa.rotate_output(pa.rotate_query(x, Pi), Pi), x, atol=1e-5)


def test_operators_refuse_cpu_tensors():
    """There is no CPU implementation behind the reference's operator names."""
    import pytest
    import torch
    import cases
    from helpers import oracle_case
    from winnow_b200 import packed_attention as pa
    c = next(x for x in cases.ATTENTION_CASES if x.name == "val_tail")
    q, okv, _ = oracle_case(c)
    kv = pa.PackedKV(okv.k_pages, okv.k_norms, okv.v_pages, okv.v_norms, okv.page_table,
                     okv.seq_lens, pa.Quantizer(okv.k_Pi, okv.k_centroids, okv.k_bits),
                     pa.Quantizer(okv.v_Pi, okv.v_centroids, okv.v_bits), c.D)
    for fn in (pa.tiled_compressed_attention, pa.explicit_compressed_attention,
               pa.reconstruct_attention):
        with pytest.raises(pa.UnsupportedLayout):
            fn(q, kv, 0.1)
