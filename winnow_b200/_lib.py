"""ctypes binding of libwinnow_tq.so.  There is no fallback: if the library is
absent or a call fails, the caller gets an exception."""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_int32, c_int64, c_size_t, c_void_p

import torch

from ._build import LIB

WTQ_F32, WTQ_F16, WTQ_BF16 = 0, 1, 2
ORDER_AUTO, ORDER_SEQUENTIAL, ORDER_INTERLEAVED16 = -1, 0, 1
STATUS_BAD_PAGE, STATUS_BAD_POSITION = 1, 2
STATUS_LAYOUT, STATUS_SCAN_TIMEOUT = 8, 16
DEQUANT_AUTO, DEQUANT_EXACT, DEQUANT_TC, DEQUANT_TC_FAST = -1, 0, 1, 2
DEQUANT_TC_MMA, DEQUANT_TC_FAST_MMA = 3, 4

_DTYPES = {torch.float32: WTQ_F32, torch.float16: WTQ_F16, torch.bfloat16: WTQ_BF16}


class BackendError(RuntimeError):
    """The CUDA library is missing, or one of its entry points refused a call."""


class Side(ctypes.Structure):
    """Mirror of wtq_side_t (include/winnow_tq.h)."""
    _fields_ = [("pages", c_void_p), ("norms", c_void_p),
                ("page_stride", c_int64), ("head_stride", c_int64),
                ("norm_page_stride", c_int64), ("norm_head_stride", c_int64),
                ("Pi", c_void_p), ("bounds", c_void_p), ("centroids", c_void_p),
                ("bw", c_int)]


class Exchange(ctypes.Structure):
    """Mirror of wtq_exchange_t (include/winnow_tq.h)."""
    _fields_ = [("peer_out", c_void_p * 2), ("peer_flags", c_void_p),
                ("out_strides", c_int64 * 2), ("rank", c_int), ("world", c_int),
                ("head_offset", c_int), ("step_counter", c_void_p), ("done_counter", c_void_p)]


STATUS_EXCHANGE_TIMEOUT = 4

_SIGNATURES = {
    "wtq_version": (c_int, []),
    "wtq_last_error": (ctypes.c_char_p, []),
    "wtq_pack": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]),
    "wtq_unpack": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]),
    "wtq_quantize": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p, c_int,
                             c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "wtq_append": (c_int, [c_void_p, c_void_p, c_int, ctypes.POINTER(c_int64),
                           ctypes.POINTER(c_int64), ctypes.POINTER(Side), ctypes.POINTER(Side),
                           c_void_p, c_int64, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                           c_int, c_int, c_void_p, c_void_p]),
    "wtq_decode_workspace_bytes": (c_size_t, [c_int] * 7),
    "wtq_decode_counter_bytes": (c_size_t, [c_int, c_int]),
    "wtq_decode_auto_splits": (c_int, [c_int] * 8),
    "wtq_decode": (c_int, [c_void_p, c_int, ctypes.POINTER(c_int64), c_void_p,
                           ctypes.POINTER(c_int64), ctypes.POINTER(Side), ctypes.POINTER(Side),
                           c_void_p, c_int64, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int,
                           c_int, c_int, c_int, c_void_p, c_size_t, c_void_p, c_void_p]),
    "wtq_launch_count": (ctypes.c_uint64, []),
    "wtq_profile_enable": (c_int, [c_int]),
    "wtq_profile_collect": (c_int, [ctypes.POINTER(ctypes.c_double), ctypes.POINTER(c_int)]),
    "wtq_profile_phases": (c_int, [ctypes.POINTER(ctypes.c_double)] * 3 + [ctypes.POINTER(c_int)]),
    "wtq_profile_disable": (c_int, []),
    "wtq_decode_exchange": (c_int, [c_void_p, c_int, ctypes.POINTER(c_int64),
                                    ctypes.POINTER(Exchange), ctypes.POINTER(Side),
                                    ctypes.POINTER(Side), c_void_p, c_int64, c_void_p, c_float,
                                    c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                    c_size_t, c_void_p, c_void_p]),
    "wtq_exchange_wait": (c_int, [c_void_p, c_int, c_void_p, c_int64, c_void_p, c_void_p]),
    "wtq_decode_exchange_supported": (c_int, [ctypes.POINTER(Side), ctypes.POINTER(Side), c_int, c_int,
                                              c_int, c_int, c_void_p]),
    "wtq_probe_read": (c_int, [c_void_p, c_size_t, c_void_p, c_void_p]),
    "wtq_decode_static_capacity": (c_size_t, []),
    "wtq_decode_static": (c_int, [c_void_p, c_int, ctypes.POINTER(c_int64), c_void_p,
                                  ctypes.POINTER(c_int64), ctypes.POINTER(Side),
                                  ctypes.POINTER(Side), c_void_p, c_int64, c_void_p, c_float,
                                  c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                  c_void_p]),
    "wtq_dense_workspace_bytes": (c_size_t, [c_int] * 4),
    "wtq_dense_decode": (c_int, [c_void_p, c_int, ctypes.POINTER(c_int64), c_void_p,
                                 ctypes.POINTER(c_int64), c_void_p, c_void_p, c_int,
                                 ctypes.POINTER(c_int64), ctypes.POINTER(c_int64), c_void_p, c_int64,
                                 c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                 c_int, c_void_p, c_size_t, c_void_p, c_void_p]),
    "wtq_prefill_auto_splits": (c_int, [c_int] * 6),
    "wtq_prefill_last_schedule": (c_int, []),
    "wtq_prefill_workspace_bytes": (c_size_t, [c_int] * 6),
    "wtq_prefill": (c_int, [c_void_p, c_int, ctypes.POINTER(c_int64), c_void_p, ctypes.POINTER(c_int64),
                            ctypes.POINTER(Side), ctypes.POINTER(Side), c_void_p, c_int64, c_void_p,
                            c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                            c_void_p, c_size_t, c_void_p, c_void_p]),
    "wtq_dequant": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                            c_int64, c_int64, c_int64, c_void_p]),
    "wtq_dequant_mode": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                 c_int, c_int64, c_int64, c_int64, c_int, c_void_p]),
}

_lib = None


def exported_symbols() -> list[str]:
    return sorted(_SIGNATURES)


def lib():
    global _lib
    if _lib is None:
        path = str(LIB)
        if not os.path.exists(path):
            raise BackendError(
                f"{LIB} is not built; run `python -c \"import __graft_entry__ as g; g.build()\"` "
                "(needs nvcc). This package has no CPU or library fallback.")
        handle = ctypes.CDLL(path)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)     # AttributeError if the symbol is missing
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        raise BackendError(f"libwinnow_tq error {rc}: {lib().wtq_last_error().decode()}")


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise BackendError(f"dtype {dtype} is not supported (float32, float16, bfloat16)") from None


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = None
    for t in tensors:
        if not t.is_cuda:
            raise BackendError(
                "the winnow_b200 operators run on CUDA tensors only; there is no CPU path")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise BackendError(f"operands on different devices: {dev} and {t.device}")
    return dev


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def i64x(*values: int):
    return (c_int64 * len(values))(*values)
