"""The CPU oracle against the golden vectors produced by the reference itself.

Everything byte- or index-valued must match bit for bit; attention outputs must
match at the reference's own CPU tolerance (2e-4, turboquant_kv/
test_packed_attention.py:22-24)."""
import numpy as np
import pytest
import torch

import cases
from helpers import digest, oracle_case
from oracle import tq_oracle as orc
from winnow_b200 import workloads


def test_codebooks_match_reference(golden):
    g = golden("codebooks")
    for D in (128, 64, 16, 8):
        for bw in orc.SUPPORTED_WIDTHS:
            if (D * bw) % 8:
                continue
            tq = orc.OracleQuantizer.get(bw, D, 42)
            assert np.array_equal(tq.centroids.numpy(), g[f"centroids_d{D}_b{bw}"]), (D, bw)
            assert np.array_equal(tq.boundaries.numpy(), g[f"boundaries_d{D}_b{bw}"]), (D, bw)
    for D in (128, 64, 16, 8):
        for seed in (42, 43):
            assert np.array_equal(orc.rotation_matrix(D, seed).numpy(), g[f"pi_d{D}_s{seed}"])


def test_known_sizes():
    assert orc.packed_bytes(128, 3) == 48 and orc.packed_bytes(128, 4) == 64
    with pytest.raises(ValueError):
        orc.packed_bytes(9, 3)


@pytest.mark.parametrize("bw", orc.SUPPORTED_WIDTHS)
def test_pack_unpack_golden(golden, bw):
    g = golden("packing")
    idx = torch.from_numpy(g[f"idx_b{bw}"])
    packed = orc.pack(idx, bw)
    assert np.array_equal(packed.numpy(), g[f"packed_b{bw}"])
    assert torch.equal(orc.unpack(packed, bw, 128), idx)
    assert torch.equal(orc.unpack_vectorized(packed, bw, 128), idx)


def test_four_bit_is_nibble_layout():
    idx = torch.arange(16, dtype=torch.uint8).repeat(8)[None]
    p = orc.pack(idx, 4)
    assert torch.equal(p, idx[:, 0::2] | (idx[:, 1::2] << 4))


@pytest.mark.parametrize("c", cases.QUANT_CASES, ids=lambda c: c.name)
def test_quantize_bit_exact(golden, c):
    g = golden("quantize")
    x = cases.quant_input(c)
    assert digest(x) == str(g[f"{c.name}/input_sha"]), "seeded input differs on this machine"
    tq = orc.OracleQuantizer.get(c.bw, c.D, 42)
    idx, norms = tq.quantize(x)
    assert np.array_equal(orc.pack(idx, c.bw).numpy(), g[f"{c.name}/packed"])
    assert np.array_equal(norms.numpy(), g[f"{c.name}/norms"])


def test_zero_vector_codes(golden):
    """A zero vector quantizes to the bucket holding 0, which is decided by the
    sign of the middle boundary: 7 at 4 bits, 32 at 6 bits."""
    for bw, code in ((4, 7), (6, 32)):
        tq = orc.OracleQuantizer.get(bw, 128, 42)
        idx, n = tq.quantize(torch.zeros(6, 128))
        assert (idx == code).all() and (n == 1e-10).all()
        assert n.to(torch.float16).eq(0).all()


def test_config1_pages_bit_exact(golden):
    g = golden("config1")
    w = workloads.WORKLOADS["config1"]
    k, v = workloads.dense_kv(w, 0)
    q = workloads.queries(w)
    assert digest(k) == str(g["k_sha"]) and digest(v) == str(g["v_sha"]) and digest(q) == str(g["q_sha"])
    kq, vq = orc.OracleQuantizer.get(4, 128, 42), orc.OracleQuantizer.get(4, 128, 43)
    kv = orc.pages_from_dense(k[None], v[None], w.seq_lens(), kq, vq, w.page_size,
                              generator=torch.Generator().manual_seed(w.seed))
    for name in ("k_pages", "v_pages", "page_table"):
        assert np.array_equal(getattr(kv, name).numpy(), g[name]), name
    for name in ("k_norms", "v_norms"):
        assert np.array_equal(getattr(kv, name).view(torch.int16).numpy(), g[name].view(np.int16)), name
    scale = orc.default_scale(128)
    for op, key in ((orc.tiled_attention, "out_tiled"), (orc.reconstruct_attention, "out_reconstruct")):
        got = op(q, kv, scale)
        assert torch.allclose(got, torch.from_numpy(g[key]), atol=2e-4, rtol=2e-4)


SMALL = [c for c in cases.ATTENTION_CASES if sum(c.lens) * c.Hkv <= 6000]


@pytest.mark.parametrize("c", SMALL, ids=lambda c: c.name)
def test_attention_matches_reference(golden, c):
    g = golden("attention")
    q, kv, _ = oracle_case(c)
    assert digest(q) == str(g[f"{c.name}/q_sha"])
    for name in ("k_pages", "k_norms", "v_pages", "v_norms", "page_table"):
        assert digest(getattr(kv, name)) == str(g[f"{c.name}/{name}_sha"]), name
    ref = torch.from_numpy(g[f"{c.name}/out"])
    scale = orc.default_scale(c.D)
    got = orc.tiled_attention(q, kv, scale)
    assert torch.allclose(got, ref, atol=2e-4, rtol=2e-4), (got - ref).abs().max()
    split = orc.tiled_attention(q, kv, scale, split_pages=2)
    assert torch.allclose(split, ref, atol=2e-4, rtol=2e-4)
    recon = orc.reconstruct_attention(q, kv, scale)
    assert torch.allclose(recon, ref, atol=2e-4, rtol=2e-4)
    for b, L in enumerate(c.lens):
        if L == 0:
            assert (got[b] == 0).all()


@pytest.mark.parametrize("c", cases.APPEND_CASES, ids=lambda c: c.name)
def test_append_matches_reference(golden, c):
    g = golden("append")
    table = torch.from_numpy(g[f"{c.name}/page_table"])
    P = cases.append_pool_pages(c)
    kq, vq = orc.OracleQuantizer.get(c.bw_k, c.D, 42), orc.OracleQuantizer.get(c.bw_v, c.D, 43)
    for layer in range(c.layers):
        kp = torch.zeros(P, c.Hkv, c.S, c.D * c.bw_k // 8, dtype=torch.uint8)
        vp = torch.zeros(P, c.Hkv, c.S, c.D * c.bw_v // 8, dtype=torch.uint8)
        kn = torch.zeros(P, c.Hkv, c.S, dtype=torch.float16)
        vn = torch.zeros(P, c.Hkv, c.S, dtype=torch.float16)
        k, v = cases.append_input(c, layer)
        orc.append_tokens(kp, kn, vp, vn, table, c.lengths, k, v, kq, vq)
        for name, t in (("k_pages", kp), ("v_pages", vp)):
            assert np.array_equal(t.numpy(), g[f"{c.name}/{name}"][layer]), (name, layer)
        for name, t in (("k_norms", kn), ("v_norms", vn)):
            assert np.array_equal(t.view(torch.int16).numpy(),
                                  g[f"{c.name}/{name}"][layer].view(np.int16)), (name, layer)
    assert np.array_equal(g[f"{c.name}/seq_lens"], np.array([L + c.n for L in c.lengths], dtype=np.int32))


@pytest.mark.parametrize("bw", [4, 6, 8, 3])
def test_dequantize_rows(golden, bw):
    g = golden("dequant")
    tq = orc.OracleQuantizer.get(bw, 128, 42)
    got = orc.dequantize_rows(torch.from_numpy(g[f"b{bw}/packed"]), torch.from_numpy(g[f"b{bw}/norms"]),
                              tq.centroids, tq.Pi, bw, 128)
    ref = torch.from_numpy(g[f"b{bw}/out_f32"])
    assert torch.allclose(got, ref, rtol=1e-5, atol=1e-6 * float(ref.abs().max()))


def test_contract_rejections():
    q, kv, _ = oracle_case(cases.ATTENTION_CASES[3])
    with pytest.raises(orc.LayoutError):
        orc.tiled_attention(q[:, :7], kv, 1.0)
    bad = orc.OracleKV(**{**kv.__dict__, "page_table": kv.page_table.clone()})
    bad.page_table[0, 0] = kv.k_pages.shape[0]
    with pytest.raises(orc.LayoutError):
        orc.tiled_attention(q, bad, 1.0)
    bad = orc.OracleKV(**{**kv.__dict__, "seq_lens": kv.seq_lens + 1000})
    with pytest.raises(orc.LayoutError):
        orc.tiled_attention(q, bad, 1.0)
