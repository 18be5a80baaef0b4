"""Chunked prefill over packed pages (wtq_prefill) against the CPU oracle.

The oracle's `tiled_attention` takes a chunk of Q query tokens per sequence,
token i seeing keys [0, seq_len - Q + i], exactly what the reference's
tiled_compressed_attention computes (turboquant_kv/packed_attention.py:260-311).
The cases cover chunk lengths 2, 16, 64 and 256, chunks longer than a
sequence's whole history (its first tokens see nothing and return zeros),
empty sequences, every width pair that has a tensor-core kernel, page sizes 16
to 64, 1 to 8 query heads per kv head, explicit and automatic chunking of the
history, the balanced schedule, query scales that push the scores beyond what fp16 score arithmetic
is trusted with, and the fallback for layouts the kernel does not serve.
"""
import pytest
import torch

from helpers import assert_attention_close, to_device
from oracle import tq_oracle as orc
from winnow_b200 import _lib, packed_attention as pa, packed_backend as pb
from winnow_b200.packed_attention_cuda import packed_prefill_attention, prefill_supported

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0) if torch.cuda.is_available() else None


def _case(seed, B, Hq, Hkv, lens, S, bw_k, bw_v, Q, q_scale=1.0, D=128):
    g = torch.Generator().manual_seed(seed)
    Lmax = max(max(lens), 1)
    k = torch.randn(B, Hkv, Lmax, D, generator=g)
    v = torch.randn(B, Hkv, Lmax, D, generator=g)
    q = torch.randn(B, Hq, Q, D, generator=g) * q_scale
    kq = orc.OracleQuantizer.get(bw_k, D, 42)
    vq = orc.OracleQuantizer.get(bw_v, D, 43)
    okv = orc.pages_from_dense(k, v, lens, kq, vq, S, generator=g)
    return q, okv


def _check(q, okv, *, splits=None, dtype=torch.float32, atol=2e-3, rel_l2=1e-3):
    scale = q.shape[-1] ** -0.5
    kv = to_device(okv, DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert prefill_supported(q.to(DEV, dtype), kv)
    before = _lib.lib().wtq_launch_count()
    out = packed_prefill_attention(q.to(DEV, dtype), kv, scale, num_splits=splits, status=status)
    assert _lib.lib().wtq_launch_count() - before == 3       # rotation, page scan, merge
    assert out.shape == q.shape and out.dtype == dtype
    ref = orc.tiled_attention(q.to(dtype).float(), okv, scale)
    assert int(status.item()) == 0
    assert_attention_close(out, ref, atol=atol, rel_l2=rel_l2)
    return out, ref


@pytest.mark.parametrize("Q", [2, 16, 64, 256])
def test_chunk_lengths_ragged_batch(Q):
    """Three sequences: one longer than the chunk, one shorter than it (its
    first tokens see no key), one of exactly one page."""
    q, okv = _case(300 + Q, 3, 14, 2, (600, max(1, Q // 2), 16), 16, 4, 4, Q)
    out, ref = _check(q, okv)
    if Q > 2:
        blind = Q - max(1, Q // 2)                            # tokens of sequence 1 before its history
        assert (out[1, :, :blind] == 0).all() and (ref[1, :, :blind] == 0).all()


@pytest.mark.parametrize("bw_k,bw_v", [(4, 4), (4, 6), (6, 6), (8, 8)])
def test_width_pairs(bw_k, bw_v):
    q, okv = _case(400 + bw_k + bw_v, 2, 8, 2, (333, 70), 16, bw_k, bw_v, 24)
    _check(q, okv)


@pytest.mark.parametrize("S,Hq,Hkv", [(16, 28, 4), (32, 8, 8), (64, 16, 2), (32, 5, 1)])
def test_page_sizes_and_head_groups(S, Hq, Hkv):
    q, okv = _case(500 + S + Hq, 2, Hq, Hkv, (270, 129), S, 4, 4, 33)
    _check(q, okv)


@pytest.mark.parametrize("splits", [1, 2, 5])
def test_history_chunking(splits):
    """Explicit split-K factors, with sequence ends inside and between chunks."""
    q, okv = _case(600 + splits, 3, 14, 2, (1500, 257, 700), 16, 4, 4, 40)
    _check(q, okv, splits=splits)


def test_empty_and_single_token_sequences():
    q, okv = _case(701, 4, 8, 2, (0, 1, 16, 17), 16, 4, 4, 8)
    out, _ = _check(q, okv)
    assert (out[0] == 0).all()


def test_bf16_queries_and_output():
    q, okv = _case(702, 2, 28, 4, (512, 100), 16, 4, 4, 64)
    _check(q, okv, dtype=torch.bfloat16, atol=2e-2, rel_l2=1e-2)   # bf16 output rounding


def test_large_scores_take_the_fp32_path():
    """Queries scaled so that scores reach the hundreds: the warps recompute
    such tiles' scores in fp32 from the packed codes."""
    q, okv = _case(703, 2, 14, 2, (200, 90), 16, 8, 8, 12, q_scale=40.0)
    _check(q, okv)
    q, okv = _case(704, 2, 8, 2, (150, 64), 16, 4, 4, 5, q_scale=25.0)
    _check(q, okv)


def test_full_chunk_of_a_long_history():
    """64 query tokens over 8k tokens of history at the benchmark's head
    geometry, one sequence (the oracle is a CPU loop)."""
    q, okv = _case(705, 1, 28, 4, (8192,), 16, 4, 4, 64)
    _check(q, okv)


@pytest.mark.parametrize("dtype,splits", [(torch.float32, 5), (torch.bfloat16, 8), (torch.float16, None),
                                          (torch.float32, 10)])
def test_many_rows_rotate_and_merge_on_the_tensor_cores(dtype, splits):
    """5120 query rows: the rotation and (up to 8 chunks per row) the merge of
    the call run as tensor-core kernels; with 10 chunks the merge falls back to
    the decode path's kernel.  Same answers either way."""
    q, okv = _case(720 + (splits or 0), 2, 32, 8, (2700, 300), 16, 4, 4, 80)
    if dtype == torch.float32:
        _check(q, okv, splits=splits)
    else:
        _check(q, okv, splits=splits, dtype=dtype, atol=2e-2, rel_l2=1e-2)


@pytest.mark.parametrize("lens,widths,dtype", [
    ((900, 0, 65, 300, 2000), (4, 4), torch.float32),        # ragged: runs of half the longest group
    ((1000,) * 10, (4, 4), torch.float32),                   # even: runs of a 148th of all tiles
    ((40, 1500, 64, 129, 700, 3), (6, 6), torch.bfloat16),   # chunks longer than some histories
    ((2100, 1, 640, 333, 70), (8, 8), torch.float16),
])
def test_balanced_schedule(lens, widths, dtype):
    """At least 74 groups and 4096 query rows: left to the library, the 64-token
    tiles of all histories are dealt evenly to the blocks, a group's pieces land
    in up to three chunk slots and rows that see nothing of a piece leave their
    slot empty.  Same answers as the oracle."""
    B, Hq, Hkv, Q = len(lens), 32, 8, 70
    q, okv = _case(740 + len(lens) + widths[0], B, Hq, Hkv, lens, 16, widths[0], widths[1], Q)
    max_pages = okv.page_table.shape[1]
    assert _lib.lib().wtq_prefill_auto_splits(B, Hq, Hkv, Q, max_pages, 16) == 3
    if dtype == torch.float32:
        out, ref = _check(q, okv)
    else:
        out, ref = _check(q, okv, dtype=dtype, atol=2e-2, rel_l2=1e-2)
    assert _lib.lib().wtq_prefill_last_schedule() == 1          # the balanced schedule did run
    for b, L in enumerate(lens):
        if L < Q:
            assert (out[b, :, :Q - L] == 0).all()                # tokens before the sequence's history
    _check(q, okv, splits=2, dtype=dtype, atol=2e-2 if dtype != torch.float32 else 2e-3,
           rel_l2=1e-2 if dtype != torch.float32 else 1e-3)
    assert _lib.lib().wtq_prefill_last_schedule() == 0          # an explicit count means equal chunks


def test_tiled_compressed_attention_uses_the_chunk_kernel():
    """The operator of the reference's name routes chunks to wtq_prefill where
    the layout allows and to B * Q decode rows where it does not."""
    q, okv = _case(706, 2, 8, 2, (90, 33), 16, 4, 4, 7)
    kv = to_device(okv, DEV)
    L = _lib.lib()
    n0 = L.wtq_launch_count()
    out = pa.tiled_compressed_attention(q.to(DEV), kv, 128 ** -0.5)
    assert L.wtq_launch_count() - n0 == 3
    assert_attention_close(out, orc.tiled_attention(q, okv, 128 ** -0.5))
    # head_dim 64 has no chunk kernel: same answer through the decode rows
    q, okv = _case(707, 2, 8, 2, (90, 33), 16, 8, 8, 7, D=64)
    kv = to_device(okv, DEV)
    assert not prefill_supported(q.to(DEV), kv)
    out = pa.tiled_compressed_attention(q.to(DEV), kv, 64 ** -0.5)
    assert_attention_close(out, orc.tiled_attention(q, okv, 64 ** -0.5))
    with pytest.raises(_lib.BackendError, match="head_dim 128"):
        packed_prefill_attention(q.to(DEV), kv, 64 ** -0.5)


def test_bad_page_id_is_reported_not_read():
    q, okv = _case(708, 2, 8, 2, (100, 40), 16, 4, 4, 9)
    kv = to_device(okv, DEV)
    kv.page_table[0, 2] = kv.k_pages.shape[0] + 5            # outside the pool
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = packed_prefill_attention(q.to(DEV), kv, 128 ** -0.5, check_page_ids=False, status=status)
    assert int(status.item()) & _lib.STATUS_BAD_PAGE
    assert torch.isfinite(out).all()
