"""Full-size benchmark workloads, checked through properties that do not need a CPU
reference of the whole thing: the split count must not change the result, the
tensor-core and generic kernels must agree, scaling the value norms scales the
output, relabelling pages leaves it unchanged, and a slice small enough for the
CPU oracle matches it."""
import os

import pytest
import torch

import bench
from helpers import assert_attention_close
from oracle import tq_oracle as orc
from winnow_b200 import packed_attention as pa, workloads
from winnow_b200.packed_attention_cuda import packed_decode_attention

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0) if torch.cuda.is_available() else None


@pytest.fixture(scope="module", params=["config2", "config3", "config4", "config5"])
def workload(request):
    w = workloads.WORKLOADS[request.param]
    if request.param == "config5":            # a quarter of the ragged batch keeps set-up short
        w = workloads.Workload(**{**w.__dict__, "batch": 32})
    pool, handles, _ = bench.build_gpu_cache(w, 0, 1, 1, DEV)
    q = workloads.queries(w).to(DEV)
    yield w, handles[0], q
    del pool, handles
    torch.cuda.empty_cache()


def test_split_count_and_kernel_choice_do_not_matter(workload, monkeypatch):
    w, kv, q = workload
    scale = w.head_dim ** -0.5
    base = packed_decode_attention(q, kv, scale, check_page_ids=False)
    # 300 and 1000 chunks per sequence only exist for the long single stream: they
    # take the merge kernel's branch for more than 256 chunks
    many = (300, 1000) if w.name == "config4" else ()
    for splits in (1, 7, 64) + many:
        other = packed_decode_attention(q, kv, scale, num_splits=splits, check_page_ids=False)
        assert_attention_close(other, base, atol=1e-3, rel_l2=5e-4)
    monkeypatch.setenv("WTQ_FORCE_GENERIC", "1")
    generic = packed_decode_attention(q, kv, scale, check_page_ids=False)
    monkeypatch.delenv("WTQ_FORCE_GENERIC")
    assert_attention_close(base, generic)


def test_value_norm_linearity_and_page_relabelling(workload):
    w, kv, q = workload
    scale = w.head_dim ** -0.5
    base = packed_decode_attention(q, kv, scale, check_page_ids=False).float()
    doubled = pa.PackedKV(**{**kv.__dict__, "v_norms": kv.v_norms * 2})
    twice = packed_decode_attention(q, doubled, scale, check_page_ids=False).float()
    assert_attention_close(twice, 2 * base, atol=4e-3)
    # move every page to a new id: same bytes, different addresses and table
    P = kv.k_pages.shape[0]
    perm = torch.randperm(P, generator=torch.Generator().manual_seed(3)).to(DEV)
    inverse = torch.empty_like(perm)
    inverse[perm] = torch.arange(P, device=DEV)
    table = kv.page_table.clone()
    used = table >= 0
    table[used] = inverse[table[used].long()].to(torch.int32)
    moved = pa.PackedKV(kv.k_pages[perm], kv.k_norms[perm], kv.v_pages[perm], kv.v_norms[perm],
                        table, kv.seq_lens, kv.k_quant, kv.v_quant, kv.head_dim)
    again = packed_decode_attention(q, moved, scale, check_page_ids=False).float()
    assert_attention_close(again, base, atol=1e-4, rel_l2=1e-4)


def test_first_sequences_match_the_oracle(workload):
    w, kv, q = workload
    scale = w.head_dim ** -0.5
    got = packed_decode_attention(q, kv, scale, check_page_ids=False)
    lens = w.seq_lens()
    short = sorted(range(w.batch), key=lambda b: lens[b])[:2]       # the two shortest sequences
    if w.name == "config4":
        short = [0]                                                  # the one long stream, whole
    for b in short:
        one = pa.PackedKV(kv.k_pages, kv.k_norms, kv.v_pages, kv.v_norms,
                          kv.page_table[b:b + 1].contiguous(), kv.seq_lens[b:b + 1].contiguous(),
                          kv.k_quant, kv.v_quant, kv.head_dim)
        okv = bench.oracle_view(w, one, 1, w.kv_heads)
        ref = orc.tiled_attention(q[b:b + 1].float().cpu(), okv, scale)
        assert_attention_close(got[b:b + 1], ref)
