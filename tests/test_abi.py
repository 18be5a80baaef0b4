"""The C-ABI library loads and exports every symbol the header declares.
No compute call is made here (there may be no GPU)."""
import ctypes
import re
from pathlib import Path

import pytest

from winnow_b200 import _build, _lib

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def library():
    if not _build.LIB.exists():
        _build.build()
    return ctypes.CDLL(str(_build.LIB))


def declared_symbols():
    text = (ROOT / "include" / "winnow_tq.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(wtq_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_entry_points():
    names = declared_symbols()
    for must in ("wtq_pack", "wtq_unpack", "wtq_quantize", "wtq_append", "wtq_decode",
                 "wtq_decode_workspace_bytes", "wtq_dequant", "wtq_last_error", "wtq_version"):
        assert must in names


def test_every_declared_symbol_is_exported(library):
    for name in declared_symbols():
        assert hasattr(library, name), f"{name} declared in include/winnow_tq.h but not exported"


def test_binding_covers_the_header():
    assert set(declared_symbols()) == set(_lib.exported_symbols())


def test_side_struct_matches_header():
    # 2 pointers, 4 int64, 3 pointers, 1 int (+ padding)
    assert ctypes.sizeof(_lib.Side) == 2 * 8 + 4 * 8 + 3 * 8 + 8


def test_argument_errors_are_reported_without_a_gpu(library):
    library.wtq_last_error.restype = ctypes.c_char_p
    library.wtq_pack.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int,
                                 ctypes.c_int, ctypes.c_void_p]
    assert library.wtq_pack(None, None, 4, 9, 3, None) == -1          # 27 bits: not whole bytes
    assert b"multiple of 8" in library.wtq_last_error()
    assert library.wtq_pack(None, None, 4, 128, 7, None) == -1        # width 7 unsupported
    assert library.wtq_pack(None, None, 0, 128, 4, None) == 0         # empty input is fine
    library.wtq_decode_workspace_bytes.restype = ctypes.c_size_t
    library.wtq_decode_workspace_bytes.argtypes = [ctypes.c_int] * 7
    small = library.wtq_decode_workspace_bytes(2, 8, 2, 128, 4, 16, 1)
    big = library.wtq_decode_workspace_bytes(2, 8, 2, 128, 4096, 16, 8)
    assert 0 < small < big


def test_auto_splits_fills_the_last_round_of_worker_warps():
    """`wtq_decode_auto_splits` is host arithmetic (148 SMs assumed without a
    GPU): for the tensor-core shapes it picks the chunk, a multiple of 32 tokens
    in [64, 1024], whose items just fill a whole number of rounds of the 1776
    worker warps (12 per SM); the answers for the benchmark shapes are pinned."""
    from winnow_b200 import _lib
    f = _lib.lib().wtq_decode_auto_splits
    workers = 148 * 12

    def items(B, Hkv, ctx, S, bk, bv, n_rep=4):
        splits = f(B, Hkv * n_rep, Hkv, 128, -(-ctx // S), S, bk, bv)
        assert 1 <= splits <= 1024
        chunk = -(-(-(-ctx // splits)) // 32) * 32
        assert 64 <= chunk <= 1024 or ctx <= 64
        return splits, B * Hkv * -(-ctx // chunk)

    assert items(16, 8, 8192, 16, 4, 4) == (13, 1664)           # config 2: one round, 94 % full
    assert items(16, 4, 8192, 16, 4, 4) == (26, 1664)           # its 2-GPU shard
    assert items(16, 1, 8192, 16, 4, 4)[0] == 86                # its 8-GPU shard: 96-token chunks
    splits, n = items(16, 8, 32768, 16, 4, 4)                   # 32k context: three rounds
    assert splits == 41 and 2.9 < n / workers <= 3.0
    assert items(1, 8, 131072, 64, 4, 4, n_rep=8) == (216, 1728)   # config 4: one round
    assert items(128, 8, 32768, 16, 4, 6)[0] == 38              # config 5: 864-token chunks
    # degenerate sizes stay in range
    assert f(1, 4, 1, 128, 1, 16, 4, 4) >= 1
    assert f(0, 4, 1, 128, 1, 16, 4, 4) == 1
    assert 1 <= f(1, 8, 1, 128, 1 << 20, 16, 4, 4) <= 1024
    # shapes without a tensor-core kernel use the generic rule and stay in range
    assert 1 <= f(4, 8, 2, 64, 64, 16, 8, 8) <= 1024


def test_prefill_planning_is_host_only(library):
    """Chunk counts and workspace sizes of the chunked-prefill entry point are
    plain host arithmetic (148 multiprocessors assumed when no GPU is present)."""
    L = _lib.lib()
    # 16 x 8 kv heads x 256 query rows: 128 groups and 32768 rows take the balanced
    # schedule (tiles dealt evenly to the blocks), three chunk states per row
    assert L.wtq_prefill_auto_splits(16, 32, 8, 64, 512, 16) == 3
    assert L.wtq_prefill_auto_splits(16, 32, 8, 256, 512, 16) == 3
    # 32 groups are too few for it: equal chunks from the cost model, 128 items in one wave
    assert L.wtq_prefill_auto_splits(4, 32, 8, 64, 512, 16) == 4
    assert L.wtq_prefill_auto_splits(1, 32, 8, 256, 8192, 16) == 4
    # one sequence: 8 groups, chunks until a wave is nearly full (144 items)
    assert L.wtq_prefill_auto_splits(1, 32, 8, 64, 8192, 16) == 18
    # a history shorter than one chunk is never split
    assert L.wtq_prefill_auto_splits(2, 8, 2, 7, 6, 16) == 1
    rows = 16 * 64 * 32
    expect = (256 + 4096 + rows * 128 * 4 + rows * 2 * 128 * 4 + 2 * rows * 2 * 4 + 256 * 256)
    assert L.wtq_prefill_workspace_bytes(16, 32, 8, 64, 128, 2) == expect
    assert L.wtq_prefill_workspace_bytes(0, 32, 8, 64, 128, 2) == 0


def test_dequant_mode_argument_errors(library):
    L = _lib.lib()
    assert L.wtq_dequant_mode(None, None, None, None, None, 2, 4, 128, 5, 5, 5, 9, None) == -1
    assert b"bad mode" in L.wtq_last_error()
    assert L.wtq_dequant_mode(None, None, None, None, None, 2, 4, 128, 0, 1, 1, _lib.DEQUANT_TC, None) == 0
    assert L.wtq_dequant_mode(None, None, None, None, None, 2, 7, 128, 4, 4, 4, _lib.DEQUANT_AUTO, None) == -1
