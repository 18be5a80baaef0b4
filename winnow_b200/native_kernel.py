"""Adapter with the call shape of the reference's native dequantization kernel
(turboquant_kv/native_kernel.py:12-40): `existing_native_kernel()` returns a
callable `(packed, norms, centroids, Pi, bit_width, head_dim, out=...)`.  The
reference looks for a prebuilt torch extension and returns None without one;
here the kernel is `wtq_dequant` of libwinnow_tq, so the adapter always exists
(and raises, as every entry point of this package does, if the library is not
built)."""
from __future__ import annotations

from .cache import dequantize_rows


def existing_native_kernel():
    """The fused dequantization kernel as a plain callable."""

    def tq_dequant_cuda(packed, norms, centroids, Pi, bit_width, head_dim, out=None):
        return dequantize_rows(packed, norms, centroids, Pi, bit_width, head_dim, out=out)

    return tq_dequant_cuda
