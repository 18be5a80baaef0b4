"""Regenerate the golden vectors under tests/golden/ from the reference itself.

Run where a checkout of the reference project is available and point
WINNOW_REFERENCE at it:

    WINNOW_REFERENCE=/path/to/winnow python tests/golden/make_golden.py

It imports the reference's own modules (packing, cache, packed_attention,
page_pool, packed_backend) read-only, runs them on the CPU on the seeded inputs
defined in tests/cases.py and winnow_b200/workloads.py, and stores what they
produce.  The tests never import the reference; they compare against these
files.  Outputs that are large are stored as SHA-256 digests.
"""
from __future__ import annotations

import hashlib
import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
REF = Path(os.environ.get("WINNOW_REFERENCE", "reference")) / "turboquant_kv"
sys.dont_write_bytecode = True
sys.path.insert(0, str(REF))
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import cache as ref_cache                      # noqa: E402  (reference)
import packed_attention as ref_pa              # noqa: E402
import packed_backend as ref_backend           # noqa: E402
import packing as ref_packing                  # noqa: E402
import page_pool as ref_pool                   # noqa: E402

import cases                                   # noqa: E402
from winnow_b200 import workloads              # noqa: E402


def digest(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def np_of(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy()
    return t.numpy()


def codebooks():
    out = {}
    for D in (128, 64, 16, 8):
        for bw in ref_packing.SUPPORTED:
            if (D * bw) % 8:
                continue
            tq = ref_cache._get_quantizer(bw, D, "cpu", 42)
            out[f"centroids_d{D}_b{bw}"] = tq.centroids.numpy()
            out[f"boundaries_d{D}_b{bw}"] = tq.boundaries.numpy()
    for D in (128, 64):
        for seed in (42, 43):
            out[f"pi_d{D}_s{seed}"] = ref_cache._get_quantizer(4, D, "cpu", seed).Pi.numpy()
    for D, seed in ((16, 42), (16, 43), (8, 42), (8, 43)):
        out[f"pi_d{D}_s{seed}"] = ref_cache._get_quantizer(8, D, "cpu", seed).Pi.numpy()
    np.savez_compressed(HERE / "codebooks.npz", **out)


def packing_vectors():
    g = torch.Generator().manual_seed(5)
    out = {}
    for bw in ref_packing.SUPPORTED:
        idx = torch.randint(0, 2 ** bw, (3, 2, 5, 128), generator=g, dtype=torch.uint8)
        idx[0, 0, 0] = 0
        idx[0, 0, 1] = 2 ** bw - 1
        out[f"idx_b{bw}"] = idx.numpy()
        out[f"packed_b{bw}"] = ref_packing.pack(idx, bw).numpy()
    np.savez_compressed(HERE / "packing.npz", **out)


def quantize_vectors():
    out = {}
    for c in cases.QUANT_CASES:
        tq = ref_cache._get_quantizer(c.bw, c.D, "cpu", 42)
        x = cases.quant_input(c)
        idx, norms = tq.quantize(x)
        out[f"{c.name}/input_sha"] = np.array(digest(x))
        out[f"{c.name}/packed"] = ref_packing.pack(idx, c.bw).numpy()
        out[f"{c.name}/norms"] = norms.numpy()
    np.savez_compressed(HERE / "quantize.npz", **out)


def attention_vectors():
    out = {}
    for c in cases.ATTENTION_CASES:
        k, v, q, g = cases.attention_inputs(c)
        kq = ref_cache._get_quantizer(c.bw_k, c.D, "cpu", 42)
        vq = ref_cache._get_quantizer(c.bw_v, c.D, "cpu", 43)
        kv = ref_pa.pages_from_dense(k, v, c.lens, kq, vq, c.S, generator=g)
        ref = ref_pa.tiled_compressed_attention(q, kv, ref_pa.default_scale(c.D))
        for name in ("k_pages", "k_norms", "v_pages", "v_norms", "page_table"):
            out[f"{c.name}/{name}_sha"] = np.array(digest(getattr(kv, name)))
        out[f"{c.name}/q_sha"] = np.array(digest(q))
        out[f"{c.name}/out"] = ref.numpy()
        print("attention", c.name, tuple(ref.shape))
    np.savez_compressed(HERE / "attention.npz", **out)


def config1_vectors():
    """Benchmark configuration 1 end to end: pages bytes, norms, table and outputs."""
    w = workloads.WORKLOADS["config1"]
    k, v = workloads.dense_kv(w, 0)
    q = workloads.queries(w)
    kq = ref_cache._get_quantizer(w.bits_k, w.head_dim, "cpu", 42)
    vq = ref_cache._get_quantizer(w.bits_v, w.head_dim, "cpu", 43)
    g = torch.Generator().manual_seed(w.seed)
    kv = ref_pa.pages_from_dense(k[None], v[None], w.seq_lens(), kq, vq, w.page_size, generator=g)
    scale = ref_pa.default_scale(w.head_dim)
    out = {"k_pages": kv.k_pages.numpy(), "v_pages": kv.v_pages.numpy(),
           "k_norms": kv.k_norms.numpy(), "v_norms": kv.v_norms.numpy(),
           "page_table": kv.page_table.numpy(),
           "k_sha": np.array(digest(k)), "v_sha": np.array(digest(v)), "q_sha": np.array(digest(q)),
           "out_tiled": ref_pa.tiled_compressed_attention(q, kv, scale).numpy(),
           "out_reconstruct": ref_pa.reconstruct_attention(q, kv, scale).numpy()}
    np.savez_compressed(HERE / "config1.npz", **out)


def append_vectors():
    """Pool contents after the reference's PagedPackedCache.update, per layer."""
    out = {}
    for c in cases.APPEND_CASES:
        P = cases.append_pool_pages(c)
        pool = ref_pool.PagePool(num_layers=c.layers, num_pages=P, num_kv_heads=c.Hkv,
                                 page_size=c.S, nb_k=c.D * c.bw_k // 8, nb_v=c.D * c.bw_v // 8)
        owners = [f"r{b}" for b in range(c.B)]
        # interleave reservations so page ids are not monotone per sequence
        for rounds in range(max(-(-(L + c.n) // c.S) for L in c.lengths)):
            for o, L in zip(reversed(owners), reversed(c.lengths)):
                pool.ensure(o, min((rounds + 1) * c.S, L + c.n))
        kq = ref_cache._get_quantizer(c.bw_k, c.D, "cpu", 42)
        vq = ref_cache._get_quantizer(c.bw_v, c.D, "cpu", 43)
        cache = ref_backend.PagedPackedCache(pool, owners, list(c.lengths), k_quant=kq, v_quant=vq,
                                             head_dim=c.D)
        for layer in range(c.layers):
            k, v = cases.append_input(c, layer)
            cache.update(k, v, layer)
        out[f"{c.name}/page_table"] = cache._table.numpy()
        out[f"{c.name}/seq_lens"] = cache._seq.numpy()
        for name in ("k_pages", "v_pages", "k_norms", "v_norms"):
            out[f"{c.name}/{name}"] = getattr(pool, name).numpy()
    np.savez_compressed(HERE / "append.npz", **out)


def dequant_vectors():
    """Fused-dequant expectation, computed as the reference's validation suite
    does (unpack, gather, @ Pi, * norm in fp32; turboquant_kv/tsc/validation.py:
    123-128) on a few of its adversarial row kinds."""
    out = {}
    g = torch.Generator().manual_seed(1103)
    for bw in (4, 6, 8, 3):
        D = 128
        tq = ref_cache._get_quantizer(bw, D, "cpu", 42)
        n = 37
        idx = torch.randint(0, 2 ** bw, (n, D), generator=g, dtype=torch.uint8)
        idx[0] = 0
        idx[1] = 2 ** bw - 1
        norms = (torch.rand(n, generator=g) * 300).half()
        norms[2], norms[3], norms[4] = 0.0, 6e-8, 6.0e4
        packed = ref_packing.pack(idx, bw)
        y = tq.centroids.index_select(0, idx.reshape(-1).long()).view(-1, D)
        x = (y @ tq.Pi) * norms.float()[:, None]
        out[f"b{bw}/packed"] = packed.numpy()
        out[f"b{bw}/norms"] = norms.numpy()
        out[f"b{bw}/out_f32"] = x.numpy()
    np.savez_compressed(HERE / "dequant.npz", **out)


if __name__ == "__main__":
    torch.set_num_threads(8)
    codebooks()
    packing_vectors()
    quantize_vectors()
    config1_vectors()
    append_vectors()
    dequant_vectors()
    attention_vectors()
    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size)
