"""Backend selection, collapsed to the one CUDA backend.

The reference plans among PyTorch, Triton and native-CUDA dequantization from
retained A6000 profiles (turboquant_kv/dispatch.py:24-244).  Here there is one
backend, built for sm_100; the planner keeps the reference's vocabulary
(`Hardware`, `Shape`, `NumericalContract`, `Decision`, `Dispatcher.select`) and
answers with that backend when the device and the shape are inside what the
library implements, and with a refusal (backend ``"none"``, never a CPU path)
otherwise.  Callers that requested a backend explicitly turn a refusal into an
error.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable

from .packing import SUPPORTED

BACKEND = "cuda_sm100"


@dataclass(frozen=True)
class Hardware:
    name: str
    compute_capability: tuple[int, int] | None

    @classmethod
    def from_torch(cls, torch_module, device) -> "Hardware":
        try:
            index = torch_module.device(device).index
            if index is None:
                index = torch_module.cuda.current_device()
            return cls(torch_module.cuda.get_device_name(index),
                       tuple(torch_module.cuda.get_device_capability(index)))
        except Exception:                              # noqa: BLE001 - no CUDA device
            return cls("unknown", None)


@dataclass(frozen=True)
class Shape:
    batch: int
    kv_heads: int
    cache_len: int
    head_dim: int
    bit_width: int

    @property
    def rows(self) -> int:
        return self.batch * self.kv_heads * self.cache_len


@dataclass(frozen=True)
class NumericalContract:
    """Largest deviation from the fp32 PyTorch reference a backend may have."""

    max_abs_error: float

    @classmethod
    def reference_exact(cls) -> "NumericalContract":
        return cls(0.0)

    @classmethod
    def quantization_aware(cls) -> "NumericalContract":
        return cls(0.03125)


@dataclass(frozen=True)
class Decision:
    backend: str
    reason: str
    estimated_speedup: float
    evidence: tuple[str, ...]


class Dispatcher:
    """One question: can the CUDA backend serve this call on this device?"""

    # fp32 accumulation throughout; measured against the fp32 reference the
    # dequant kernel differs by summation order only.
    BACKEND_MAX_ABS_ERROR = 1e-5

    def __init__(self):
        self._cache: dict[tuple, Decision] = {}

    def select(self, hardware: Hardware, shape: Shape, contract: NumericalContract,
               available: Iterable[str] = (BACKEND,)) -> Decision:
        key = (hardware, shape, contract, frozenset(available))
        hit = self._cache.get(key)
        if hit is not None:
            return hit
        cc = hardware.compute_capability
        if cc is None or cc[0] != 10:
            d = Decision("none", f"{hardware.name} is not an sm_100 device; no other backend exists",
                         1.0, ())
        elif BACKEND not in key[3]:
            d = Decision("none", "the CUDA library is not available", 1.0, ())
        elif shape.bit_width not in SUPPORTED or (shape.head_dim * shape.bit_width) % 8 \
                or not 1 <= shape.head_dim <= 256:
            d = Decision("none", f"head_dim {shape.head_dim} at {shape.bit_width} bits is outside "
                         "the library's envelope", 1.0, ())
        elif contract.max_abs_error < self.BACKEND_MAX_ABS_ERROR:
            d = Decision("none", "error budget below fp32 summation-order noise", 1.0, ())
        else:
            d = Decision(BACKEND, "single CUDA backend, fp32 accumulation", 1.0,
                         ("profiles/",))
        self._cache[key] = d
        return d


_DEFAULT: Dispatcher | None = None


def default_dispatcher() -> Dispatcher:
    global _DEFAULT
    if _DEFAULT is None:
        _DEFAULT = Dispatcher()
    return _DEFAULT
