"""Bit-packing of codebook indices on the GPU.

Same layout contract as the reference (turboquant_kv/packing.py:14-18,38-89):
LSB-first within an index, indices in order along the last axis, an index may
straddle a byte; 4-bit is therefore byte i = idx[2i] | idx[2i+1] << 4.
"""
from __future__ import annotations

import torch

from . import _lib

SUPPORTED = (2, 3, 4, 5, 6, 8)


def packed_bytes(head_dim: int, bit_width: int) -> int:
    """Bytes one `head_dim`-long vector of `bit_width`-bit indices occupies."""
    total_bits = head_dim * bit_width
    if total_bits % 8 != 0:
        raise ValueError(f"head_dim*bit_width must be a multiple of 8, got "
                         f"{head_dim}*{bit_width}={total_bits}")
    return total_bits // 8


def _check_width(bit_width: int) -> None:
    if bit_width not in SUPPORTED:
        raise ValueError(f"bit_width {bit_width} not in {SUPPORTED}")


@torch.no_grad()
def pack(idx: torch.Tensor, bit_width: int) -> torch.Tensor:
    """(..., D) uint8 indices -> (..., D*bit_width/8) uint8."""
    _check_width(bit_width)
    if idx.dtype != torch.uint8:
        raise ValueError("indices must be uint8")
    if bit_width == 8:
        return idx.contiguous()
    dev = _lib.require_cuda(idx)
    D = idx.shape[-1]
    nb = packed_bytes(D, bit_width)
    src = idx.contiguous()
    out = torch.empty(*idx.shape[:-1], nb, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().wtq_pack(src.data_ptr(), out.data_ptr(), src.numel() // D, D,
                                       bit_width, _lib.stream_ptr(dev)))
    return out


@torch.no_grad()
def unpack(packed: torch.Tensor, bit_width: int, head_dim: int) -> torch.Tensor:
    """(..., D*bit_width/8) uint8 -> (..., D) uint8 indices."""
    _check_width(bit_width)
    if packed.dtype != torch.uint8:
        raise ValueError("packed rows must be uint8")
    if bit_width == 8:
        return packed
    nb = packed_bytes(head_dim, bit_width)
    if packed.shape[-1] != nb:
        raise ValueError(f"rows of {packed.shape[-1]} bytes do not hold {head_dim} {bit_width}-bit codes")
    dev = _lib.require_cuda(packed)
    src = packed.contiguous()
    out = torch.empty(*packed.shape[:-1], head_dim, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().wtq_unpack(src.data_ptr(), out.data_ptr(), src.numel() // nb,
                                         head_dim, bit_width, _lib.stream_ptr(dev)))
    return out
