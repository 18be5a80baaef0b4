"""Shared helpers of the test-suite: digests, oracle fixtures, device copies."""
from __future__ import annotations

import hashlib

import torch

import cases
from oracle import tq_oracle as orc

ATOL = 2e-3           # max-abs bound on attention outputs (fp32 accumulation)
REL_L2 = 1e-3         # relative L2 bound


def digest(t: torch.Tensor) -> str:
    return hashlib.sha256(t.detach().cpu().contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def oracle_case(c: cases.AttnCase):
    """q and the oracle's paged cache for a frozen attention case."""
    k, v, q, g = cases.attention_inputs(c)
    kq = orc.OracleQuantizer.get(c.bw_k, c.D, 42)
    vq = orc.OracleQuantizer.get(c.bw_v, c.D, 43)
    kv = orc.pages_from_dense(k, v, c.lens, kq, vq, c.S, generator=g)
    return q, kv, (k, v)


def to_device(kv: orc.OracleKV, dev):
    """The package's PackedKV on `dev` holding the oracle's bytes."""
    from winnow_b200 import packed_attention as pa
    return pa.PackedKV(kv.k_pages.to(dev), kv.k_norms.to(dev), kv.v_pages.to(dev),
                       kv.v_norms.to(dev), kv.page_table.to(dev), kv.seq_lens.to(dev),
                       pa.Quantizer(kv.k_Pi.to(dev), kv.k_centroids.to(dev), kv.k_bits),
                       pa.Quantizer(kv.v_Pi.to(dev), kv.v_centroids.to(dev), kv.v_bits),
                       kv.head_dim)


def assert_attention_close(got: torch.Tensor, ref: torch.Tensor, atol=ATOL, rel_l2=REL_L2):
    got, ref = got.float().cpu(), ref.float().cpu()
    assert torch.isfinite(got).all()
    err = (got - ref).abs().max().item()
    assert err <= atol, f"max abs err {err:.3e} > {atol}"
    denom = ref.norm().item()
    if denom > 0:
        rel = (got - ref).norm().item() / denom
        assert rel <= rel_l2, f"relative L2 {rel:.3e} > {rel_l2}"
