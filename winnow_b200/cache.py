"""TurboQuant quantizer: fixed random rotation + Lloyd-Max scalar codebook.

Construction (rotation by QR of a CPU-seeded Gaussian matrix, codebook by
Lloyd-Max iteration in float64) runs once per (bit width, head_dim, seed) on the
host and defines the codebook bit for bit, as in the reference
(turboquant_kv/cache.py:62-106,134-148).  `quantize` and `dequantize_into` run
on the GPU through libwinnow_tq.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from . import _lib
from .packing import packed_bytes


def _lloyd_max_gaussian(levels: int, sigma: float = 1.0, iters: int = 200, tol: float = 1e-12):
    """Lloyd-Max centroids and bucket edges (with the +-inf ends) for
    N(0, sigma^2), float64.  Evenly spaced start on [-3 sigma, 3 sigma]; edges
    midway between neighbours; centroids to the conditional mean of their bucket;
    stop when no centroid moves more than `tol`."""
    from scipy.stats import norm

    c = np.linspace(-3.0 * sigma, 3.0 * sigma, levels)
    for _ in range(iters):
        z = np.concatenate(([-np.inf], 0.5 * (c[:-1] + c[1:]), [np.inf])) / sigma
        mass = norm.cdf(z[1:]) - norm.cdf(z[:-1])
        first_moment = sigma * (norm.pdf(z[:-1]) - norm.pdf(z[1:]))
        with np.errstate(divide="ignore", invalid="ignore"):
            nxt = np.where(mass < 1e-300, c, first_moment / mass)
        converged = np.max(np.abs(nxt - c)) < tol
        c = nxt
        if converged:
            break
    return c, np.concatenate(([-np.inf], 0.5 * (c[:-1] + c[1:]), [np.inf]))


class TurboQuantMSE:
    """Pi (D, D) fp32, centroids (2^bw) fp32, boundaries (2^bw - 1) fp32."""

    def __init__(self, bit_width: int, head_dim: int, device="cpu", rotation_seed: int = 42):
        packed_bytes(head_dim, bit_width)
        device = torch.device(device)
        gen = torch.Generator(device="cpu").manual_seed(rotation_seed)
        gauss = torch.randn(head_dim, head_dim, generator=gen, dtype=torch.float32)
        Q, R = torch.linalg.qr(gauss)
        signs = torch.sign(torch.diag(R))
        signs[signs == 0] = 1.0
        self.Pi = (Q * signs.unsqueeze(0)).to(device).contiguous()
        c, edges = _lloyd_max_gaussian(2 ** bit_width, sigma=1.0 / math.sqrt(head_dim))
        self.centroids = torch.tensor(c, dtype=torch.float32, device=device).contiguous()
        self.boundaries = torch.tensor(edges[1:-1], dtype=torch.float32, device=device).contiguous()
        self.bit_width, self.head_dim, self.device = bit_width, head_dim, device

    @torch.no_grad()
    def quantize(self, x: torch.Tensor, *, order: int = _lib.ORDER_AUTO, packed: bool = False):
        """(..., D) -> (uint8 idx (..., D), fp32 norms (...,)).

        With `packed=True` the first result is the bit-packed rows
        (..., D*bw/8) instead, produced by the same launch.  `order` selects the
        summation order of the rotation (see include/winnow_tq.h); the default
        follows the reference's CPU arithmetic for this many vectors.
        """
        D = self.head_dim
        if x.shape[-1] != D:
            raise ValueError(f"last dimension {x.shape[-1]} != head_dim {D}")
        dev = _lib.require_cuda(x, self.Pi)
        src = x if x.dtype in (torch.float32, torch.float16, torch.bfloat16) else x.float()
        src = src.reshape(-1, D)
        if src.stride(-1) != 1:
            src = src.contiguous()
        rows = src.shape[0]
        nb = packed_bytes(D, self.bit_width)
        codes = torch.empty(*x.shape[:-1], nb if packed else D, dtype=torch.uint8, device=dev)
        norms = torch.empty(x.shape[:-1], dtype=torch.float32, device=dev)
        if rows:
            with torch.cuda.device(dev):
                _lib.check(_lib.lib().wtq_quantize(
                    src.data_ptr(), _lib.dtype_code(src.dtype), rows, src.stride(0), D,
                    self.Pi.data_ptr(), self.boundaries.data_ptr(), self.bit_width, order,
                    None if packed else codes.data_ptr(), codes.data_ptr() if packed else None,
                    norms.data_ptr(), _lib.stream_ptr(dev)))
        return codes, norms

    @torch.no_grad()
    def dequantize_into(self, idx: torch.Tensor, norms: torch.Tensor, out: torch.Tensor) -> None:
        """Reconstruct `centroids[idx] @ Pi * norms` into `out` (fp32/fp16/bf16)."""
        from .packing import pack
        rows = pack(idx.reshape(-1, self.head_dim), self.bit_width)
        dequantize_rows(rows, norms.reshape(-1).to(torch.float16), self.centroids, self.Pi,
                        self.bit_width, self.head_dim, out=out)


@torch.no_grad()
def dequantize_rows(packed: torch.Tensor, norms: torch.Tensor, centroids: torch.Tensor,
                    Pi: torch.Tensor, bit_width: int, head_dim: int,
                    out: torch.Tensor | None = None, allow_tf32: bool = False,
                    mode: str | None = None) -> torch.Tensor:
    """Fused dequantisation of packed rows, the counterpart of the reference's
    `tq_dequant` (turboquant_kv/kernel.py:78-115).

    `packed` is (..., NB) uint8 and `norms` (...,) fp16.  A (B, H, L, NB) slice
    of a (B, H, MAXLEN, NB) buffer is read in place through its strides.
    Returns (..., head_dim) in `out`'s dtype (bf16 when `out` is None).

    Arithmetic (`mode`): "exact" is an fp32 contraction on the CUDA cores; "tc"
    runs on the tensor cores with centroids and Pi split into fp16 high and low
    parts (three products, fp32 accumulation); "tc_fast" uses single fp16
    operands, the accuracy class of the reference's `allow_tf32=True`; both run
    the tcgen05 kernel (accumulator in tensor memory), "tc_mma" / "tc_fast_mma"
    name the mma.sync kernels they fall back to.  With
    `mode=None`: `allow_tf32=True` asks for "tc_fast" where the tensor-core
    kernel applies (head_dim 128, widths 4/6/8), otherwise the library picks
    "tc" for 16-bit outputs it applies to and "exact" for everything else.
    """
    if mode is None:
        code = _lib.DEQUANT_AUTO
        if allow_tf32 and head_dim == 128 and bit_width in (4, 6, 8):
            code = _lib.DEQUANT_TC_FAST
    else:
        code = {"exact": _lib.DEQUANT_EXACT, "tc": _lib.DEQUANT_TC, "tc_fast": _lib.DEQUANT_TC_FAST,
                "tc_mma": _lib.DEQUANT_TC_MMA, "tc_fast_mma": _lib.DEQUANT_TC_FAST_MMA}[mode]
    dev = _lib.require_cuda(packed, norms, centroids, Pi)
    nb = packed_bytes(head_dim, bit_width)
    if packed.dtype != torch.uint8 or packed.shape[-1] != nb:
        raise ValueError(f"packed rows must be uint8 with {nb} bytes")
    if norms.dtype != torch.float16:
        raise ValueError("norms must be fp16")
    lead = packed.shape[:-1]
    N = 1
    for s in lead:
        N *= s
    L = lead[-1] if lead else 1
    maxlen = L
    src, nsrc = packed, norms
    if (packed.dim() >= 3 and not packed.is_contiguous() and _is_plane_slice(packed, nb)
            and _is_plane_slice(norms.unsqueeze(-1), 1)
            and norms.stride(-2) * nb == packed.stride(-3)):
        maxlen = packed.stride(-3) // nb
    elif not packed.is_contiguous() or not norms.is_contiguous():
        src, nsrc = packed.contiguous(), norms.contiguous()
    if out is None:
        out = torch.empty(*lead, head_dim, dtype=torch.bfloat16, device=dev)
    if not out.is_contiguous() or out.numel() != N * head_dim:
        raise ValueError("out must be contiguous with shape (..., head_dim)")
    if N:
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().wtq_dequant_mode(
                src.data_ptr(), nsrc.data_ptr(), centroids.data_ptr(), Pi.data_ptr(),
                out.data_ptr(), _lib.dtype_code(out.dtype), bit_width, head_dim, N, L, maxlen,
                code, _lib.stream_ptr(dev)))
    return out


def _is_plane_slice(t: torch.Tensor, row: int) -> bool:
    """True when `t` (..., L, row) is the first-L-positions view of a dense
    (..., MAXLEN, row) buffer: the leading dimensions are contiguous over planes
    of MAXLEN rows."""
    if t.stride(-1) != 1 or t.stride(-2) != row:
        return False
    plane = t.stride(-3)
    if plane % row or plane < t.shape[-2] * row:
        return False
    expect = plane
    for size, stride in zip(reversed(t.shape[:-2]), reversed(t.stride()[:-2])):
        if size != 1 and stride != expect:
            return False
        expect *= size
    return True


_QUANTIZER_CACHE: dict = {}


def _get_quantizer(bw, dim, dev, seed=42) -> TurboQuantMSE:
    """One quantizer per (bit width, head_dim, device, seed); building one costs
    a scipy iteration, and every layer of a model shares it."""
    key = (bw, dim, str(dev), seed)
    if key not in _QUANTIZER_CACHE:
        _QUANTIZER_CACHE[key] = TurboQuantMSE(bw, dim, dev, rotation_seed=seed)
    return _QUANTIZER_CACHE[key]


try:                                      # the legacy cache is an HF cache when transformers is present
    from transformers.cache_utils import DynamicCache as _CacheBase, DynamicLayer as _LayerBase
except Exception:                         # noqa: BLE001 - optional dependency
    _CacheBase = _LayerBase = object


class TQPackedLayer(_LayerBase):
    """Contiguous packed KV of one layer: a preallocated (B, H, max_len, NB) ring
    of codes plus fp16 norms, written in place, and a transient dequantization
    of the whole history per step (reference: turboquant_kv/cache.py:154-373).
    A `transformers` `DynamicLayer` when that package is importable, as the
    reference's class is, so it can sit in a `past_key_values` cache.

    This is the legacy cache of the reference: it hands dense K, V to stock
    attention, so its decode cost grows with the history.  The paged cache with
    compressed-domain attention (packed_backend.PagedPackedCache) is the path
    to use; this class exists for callers that still hold the old interface.
    Both directions run on the GPU: `wtq_quantize` with fused packing for the
    write, `wtq_dequant` reading the ring in place for the read.

    Outlier channels (turboquant_kv/cache.py:183-191,224-233,289-303): with
    `num_outlier_channels` > 0 and `outlier_bits` > `bit_width`, the channels
    with the largest RMS in the first keys seen go to a second quantizer
    (`outlier_bits` wide, rotation seed 43) over just those channels, the rest
    to the regular one over the remaining channels; each part has its own codes
    and norms, and the read scatters the two reconstructions back into place.
    The keyword arguments that chose among the reference's dequantization
    back-ends (`chunk`, `use_kernel`, `allow_tf32`, `kernel_backend`,
    `native_kernel`) are accepted and ignored: there is one back-end here.
    """

    def __init__(self, head_dim: int, bit_width: int, device, max_cache_len: int,
                 num_outlier_channels: int = 0, outlier_bits: int = 0, chunk: int = 1024,
                 use_kernel: bool = True, allow_tf32: bool = True, kernel_backend: str = "auto",
                 native_kernel=None, dispatcher=None):
        if _LayerBase is not object:
            super().__init__()
        del chunk, use_kernel, allow_tf32, native_kernel
        if kernel_backend not in {"auto", "torch_fp32", "triton_fp32", "triton_tf32",
                                  "native_cuda_fp32", "cuda_sm100"}:
            raise ValueError(f"unknown kernel_backend={kernel_backend!r}")
        self._dispatcher = dispatcher
        self._bw, self._hd, self._max = bit_width, head_dim, max_cache_len
        split = num_outlier_channels > 0 and outlier_bits > bit_width
        self._out_dim = num_outlier_channels if split else 0
        self._reg_dim = head_dim - self._out_dim
        self._out_bw = outlier_bits
        self._tq = _get_quantizer(bit_width, self._reg_dim, device)
        self._tq_out = _get_quantizer(outlier_bits, self._out_dim, device, seed=43) if split else None
        self._nb = packed_bytes(self._reg_dim, bit_width)
        self._nb_out = packed_bytes(self._out_dim, outlier_bits) if split else 0
        self._len = 0
        self._channels = None               # (regular channel ids, outlier channel ids)
        self.is_initialized = False
        self.last_dispatch_decision = None

    def lazy_initialization(self, ks: torch.Tensor, vs: torch.Tensor) -> None:
        from .dispatch import Hardware, NumericalContract, Shape, default_dispatcher
        B, H, _, D = ks.shape
        dev = _lib.require_cuda(ks, vs)
        self.dtype, self.device = ks.dtype, dev

        def ring(nb):
            return torch.empty(B, H, self._max, nb, dtype=torch.uint8, device=dev)

        def norms():
            return torch.empty(B, H, self._max, dtype=torch.float16, device=dev)

        # per tensor (K, V): [regular codes, regular norms, outlier codes, outlier norms]
        self._k = [ring(self._nb), norms(), None, None]
        self._v = [ring(self._nb), norms(), None, None]
        if self._out_dim:
            for side in (self._k, self._v):
                side[2], side[3] = ring(self._nb_out), norms()
            rms = ks.float().pow(2).mean(dim=(0, 1, 2)).sqrt()
            top = rms.topk(min(self._out_dim, D)).indices
            mask = torch.zeros(D, dtype=torch.bool, device=dev)
            mask[top] = True
            self._mask = mask
            self._channels = ((~mask).nonzero().flatten(), mask.nonzero().flatten())
        self._shape = (B, H, D)
        self.last_dispatch_decision = (self._dispatcher or default_dispatcher()).select(
            Hardware.from_torch(torch, dev), Shape(B, H, self._max, D, self._bw),
            NumericalContract.quantization_aware())
        if self.last_dispatch_decision.backend == "none":
            raise _lib.BackendError(self.last_dispatch_decision.reason)
        self.is_initialized = True

    def _store(self, x, pos, n, side):
        parts = ((self._tq, None, 0),) if not self._out_dim else (
            (self._tq, self._channels[0], 0), (self._tq_out, self._channels[1], 2))
        for tq, channels, at in parts:
            src = x if channels is None else x.float().index_select(-1, channels)
            packed, nrm = tq.quantize(src, packed=True)
            side[at][:, :, pos:pos + n] = packed
            side[at + 1][:, :, pos:pos + n] = nrm.to(torch.float16)

    def _load(self, length, side):
        B, H, D = self._shape
        out = torch.empty(B, H, length, D, dtype=self.dtype, device=self.device)
        if not self._out_dim:
            return dequantize_rows(side[0][:, :, :length], side[1][:, :, :length],
                                   self._tq.centroids, self._tq.Pi, self._bw, D, out=out)
        for tq, channels, at, bw, dim in ((self._tq, self._channels[0], 0, self._bw, self._reg_dim),
                                          (self._tq_out, self._channels[1], 2, self._out_bw,
                                           self._out_dim)):
            part = torch.empty(B, H, length, dim, dtype=self.dtype, device=self.device)
            dequantize_rows(side[at][:, :, :length], side[at + 1][:, :, :length], tq.centroids,
                            tq.Pi, bw, dim, out=part)
            out.index_copy_(-1, channels, part)
        return out

    @torch.no_grad()
    def update(self, key_states, value_states, *args, **kwargs):
        if not self.is_initialized:
            self.lazy_initialization(key_states, value_states)
        n = key_states.shape[-2]
        if self._len + n > self._max:
            raise RuntimeError(f"TQPackedLayer overflow: {self._len}+{n} > max_cache_len="
                               f"{self._max}. Raise max_cache_len.")
        self._store(key_states, self._len, n, self._k)
        self._store(value_states, self._len, n, self._v)
        self._len += n
        return self._load(self._len, self._k), self._load(self._len, self._v)

    # ---- cache protocol ----------------------------------------------------------
    def get_seq_length(self, *args, **kwargs) -> int:
        return self._len

    def get_mask_sizes(self, query_length: int = 0, *args, **kwargs):
        return self._len, 0

    def get_max_length(self, *args, **kwargs):
        return self._max

    def get_max_cache_shape(self, *args, **kwargs):
        return self._max

    def reset(self):
        self._len = 0

    # ---- accounting --------------------------------------------------------------
    def _tensors(self):
        if not self.is_initialized:
            return []
        return [t for side in (self._k, self._v) for t in side if t is not None]

    def persistent_bytes(self) -> int:
        """Bytes this layer holds between steps (codes + norms for the whole ring)."""
        return sum(t.numel() * t.element_size() for t in self._tensors())

    packed_bytes_held = persistent_bytes

    def persistent_bytes_used(self) -> int:
        """The same, counting only the positions written so far."""
        return int(self.persistent_bytes() * self._len / self._max) if self._max else 0

    def transient_bytes(self) -> int:
        """Bytes of the dequantized K and V handed to attention this step."""
        if not self.is_initialized:
            return 0
        B, H, D = self._shape
        return 2 * B * H * self._len * D * torch.empty((), dtype=self.dtype).element_size()


class TQPackedCache(_CacheBase):
    """`past_key_values` made of `TQPackedLayer`s (reference:
    turboquant_kv/cache.py:376-419): `TQPackedCache(config, bit_width,
    max_cache_len, device=...)` as there, or, without a model config,
    `TQPackedCache(head_dim, bit_width, device, max_cache_len, num_layers)`."""

    def __init__(self, config_or_head_dim, bit_width: int, *args, **kwargs):
        if _CacheBase is not object:
            super().__init__()
        if hasattr(config_or_head_dim, "num_hidden_layers"):
            cfg = config_or_head_dim
            head_dim = getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads
            num_layers = cfg.num_hidden_layers
            max_cache_len = args[0] if args else kwargs.pop("max_cache_len")
            device = args[1] if len(args) > 1 else kwargs.pop("device", "cuda")
        else:
            head_dim = int(config_or_head_dim)
            device = args[0] if args else kwargs.pop("device")
            max_cache_len = args[1] if len(args) > 1 else kwargs.pop("max_cache_len")
            num_layers = args[2] if len(args) > 2 else kwargs.pop("num_layers")
        self.layers = [TQPackedLayer(head_dim, bit_width, device, max_cache_len, **kwargs)
                       for _ in range(num_layers)]
        self.bit_width, self.head_dim = bit_width, head_dim
        self.append_new_layers = lambda *a, **k: None

    def update(self, key_states, value_states, layer_idx: int, *args, **kwargs):
        return self.layers[layer_idx].update(key_states, value_states)

    def get_seq_length(self, layer_idx: int = 0, *args, **kwargs) -> int:
        return self.layers[layer_idx].get_seq_length()

    def persistent_bytes(self) -> int:
        return sum(layer.persistent_bytes() for layer in self.layers)

    def persistent_bytes_used(self) -> int:
        return sum(layer.persistent_bytes_used() for layer in self.layers)

    def transient_bytes(self) -> int:
        return max((layer.transient_bytes() for layer in self.layers), default=0)

    def effective_bits(self) -> float:
        """Stored bits per KV element, norms included."""
        layer = self.layers[0]
        if not layer.is_initialized:
            return float("nan")
        bits = 8 * (layer._nb + layer._nb_out) + 16 * (2 if layer._out_dim else 1)
        return bits / self.head_dim
