"""Decode attention over paged packed K/V on the CUDA backend.

Counterpart of the reference's Triton operator
(turboquant_kv/packed_attention_triton.py:166-262) with its call signature:
one query token per sequence, `q` (B, Hq, 1, D) in any float dtype, result
(B, Hq, 1, D) in `q.dtype`, fp32 inside.  The query rotation, the split-K scan
of the page table and the merge with the output rotation all run inside
libwinnow_tq (wtq_decode); the only allocations are the result and one
workspace whose size depends on batch, heads and splits, never on history
length.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from . import packed_attention as pa


def check_kernel_contract(q: torch.Tensor, kv: pa.PackedKV, *, check_page_ids: bool = True) -> None:
    pa.check_contract(q, kv, check_page_ids=check_page_ids)
    if q.shape[2] != 1:
        raise pa.UnsupportedLayout("the CUDA decode kernel serves one query token per sequence")
    if not q.is_cuda:
        raise pa.UnsupportedLayout("the CUDA decode kernel needs CUDA tensors")
    if q.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise pa.UnsupportedLayout(f"q dtype {q.dtype} is not a supported float type")
    if kv.head_dim > 256:
        raise pa.UnsupportedLayout("head_dim above 256 is not supported")
    for name, pages, norms in (("k", kv.k_pages, kv.k_norms), ("v", kv.v_pages, kv.v_norms)):
        if pages.stride(-1) != 1 or pages.stride(-2) != pages.shape[-1] or norms.stride(-1) != 1:
            raise pa.UnsupportedLayout(f"{name} pages need contiguous (S, NB) rows and contiguous "
                                       "norm slots")
    if kv.page_table.stride(-1) != 1 or not kv.seq_lens.is_contiguous():
        raise pa.UnsupportedLayout("page_table rows and seq_lens must be contiguous")
    for quant in (kv.k_quant, kv.v_quant):
        if not quant.Pi.is_contiguous() or not quant.centroids.is_contiguous():
            raise pa.UnsupportedLayout("rotations and codebooks must be contiguous")


def _side(pages, norms, quant, bounds=None) -> _lib.Side:
    return _lib.Side(pages.data_ptr(), norms.data_ptr(), pages.stride(0), pages.stride(1),
                     norms.stride(0), norms.stride(1), quant.Pi.data_ptr(),
                     bounds.data_ptr() if bounds is not None else None,
                     quant.centroids.data_ptr() if quant.centroids is not None else None,
                     quant.bit_width)


def decode_workspace(B: int, Hq: int, Hkv: int, D: int, max_pages: int, S: int,
                     num_splits: int, device) -> torch.Tensor:
    """Workspace for one call; its leading counter block starts zeroed."""
    L = _lib.lib()
    size = L.wtq_decode_workspace_bytes(B, Hq, Hkv, D, max_pages, S, num_splits)
    ws = torch.empty(size, dtype=torch.uint8, device=device)
    ws[: L.wtq_decode_counter_bytes(B, Hkv)].zero_()
    return ws


class DecodePlan:
    """One decode call with every argument marshalled ahead of time.

    A serving loop calls the operator with the same tensors step after step
    (the page table, lengths, query and output buffers are updated in place),
    so the contract checks and the ctypes marshalling are done once here and
    `run()` is a single call into the library on the current stream.  The plan
    keeps its tensors alive.  `graph()` captures the call's launches into a
    CUDA graph for replay.
    """

    def __init__(self, q: torch.Tensor, kv: pa.PackedKV, scale: float, *,
                 num_splits: int | None = None, out: torch.Tensor | None = None,
                 workspace: torch.Tensor | None = None, status: torch.Tensor | None = None,
                 check_page_ids: bool = True):
        check_kernel_contract(q, kv, check_page_ids=check_page_ids)
        B, Hq, _, D = q.shape
        dev = q.device
        Hkv, S, P = kv.num_kv_heads, kv.page_size, kv.k_pages.shape[0]
        max_pages = kv.page_table.shape[1]
        if q.stride(-1) != 1:
            raise pa.UnsupportedLayout("q must have unit stride in its last dimension")
        if out is None:
            out = torch.empty(B, Hq, 1, D, dtype=q.dtype, device=dev)
        elif tuple(out.shape) != (B, Hq, 1, D) or out.dtype != q.dtype or out.stride(-1) != 1 \
                or out.device != dev:
            raise pa.UnsupportedLayout("out must be (B, Hq, 1, D) in q.dtype with unit stride in D")
        self.out, self.device = out, dev
        self.empty = B == 0 or max_pages == 0
        if self.empty:
            return
        splits = int(num_splits or 0)
        if workspace is None:
            workspace = decode_workspace(B, Hq, Hkv, D, max_pages, S, splits, dev)
        self._keep = (q, kv, out, workspace, status)
        self._k_side = _side(kv.k_pages, kv.k_norms, kv.k_quant)
        self._v_side = _side(kv.v_pages, kv.v_norms, kv.v_quant)
        self._qs = _lib.i64x(q.stride(0), q.stride(1))
        self._os = _lib.i64x(out.stride(0), out.stride(1))
        self._fn = _lib.lib().wtq_decode
        self._args = (
            q.data_ptr(), _lib.dtype_code(q.dtype), self._qs, out.data_ptr(), self._os,
            ctypes.byref(self._k_side), ctypes.byref(self._v_side),
            kv.page_table.data_ptr(), kv.page_table.stride(0), kv.seq_lens.data_ptr(),
            float(scale), B, Hq, Hkv, D, S, P, max_pages, splits,
            workspace.data_ptr(), workspace.numel(),
            status.data_ptr() if status is not None else None)

    def run(self) -> torch.Tensor:
        if self.empty:
            return self.out.zero_() if self.out.numel() else self.out
        stream = torch.cuda.current_stream(self.device).cuda_stream
        rc = self._fn(*self._args, stream)
        if rc:
            _lib.check(rc)
        return self.out

    def run_exchange(self, exchange, dry_run: bool = False):
        """The call with its output exchange fused (`wtq_decode_exchange`):
        `exchange` is a `_lib.Exchange` descriptor naming every rank's buffers.
        `dry_run` only asks the library whether this shape has the fused
        epilogue (raises `BackendError` if not) without launching anything."""
        a = self._args
        if dry_run:
            ok = _lib.lib().wtq_decode_exchange_supported(
                ctypes.byref(self._k_side), ctypes.byref(self._v_side), a[12], a[13], a[14], a[15],
                a[19])
            if not ok:
                raise _lib.BackendError("no fused exchange epilogue for this shape")
            return None
        stream = torch.cuda.current_stream(self.device).cuda_stream
        if not hasattr(self, "_fn_exchange"):
            self._fn_exchange = _lib.lib().wtq_decode_exchange
        rc = self._fn_exchange(a[0], a[1], a[2], ctypes.byref(exchange), *a[5:], stream)
        if rc:
            _lib.check(rc)
        return None

    def graph(self) -> "torch.cuda.CUDAGraph":
        """The call captured as a CUDA graph (replay with `.replay()`)."""
        with torch.cuda.device(self.device):
            self.run()                                   # first call: one-time attribute set-up
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.run()
        return g


@torch.no_grad()
def packed_decode_attention(q: torch.Tensor, kv: pa.PackedKV, scale: float, *,
                            num_splits: int | None = None, allow_tf32: bool = False,
                            num_warps: int = 4, num_stages: int = 2, pages_per_iter: int = 1,
                            check_page_ids: bool = True, out: torch.Tensor | None = None,
                            workspace: torch.Tensor | None = None,
                            status: torch.Tensor | None = None) -> torch.Tensor:
    """q (B, Hq, 1, D) -> (B, Hq, 1, D) in q.dtype.

    `num_splits=None` (or 0) lets the backend size the split-K grid; a positive
    value is honoured.  `allow_tf32`, `num_warps`, `num_stages` and
    `pages_per_iter` are accepted for call compatibility with the Triton
    operator; only `pages_per_iter` is validated (a power of two), none changes
    the CUDA schedule.  `out` may be a (B, Hq, 1, D) view into a larger buffer
    (e.g. this rank's heads inside a gathered output) with unit stride in D.
    """
    if pages_per_iter < 1 or pages_per_iter & (pages_per_iter - 1):
        pa.check_contract(q, kv, check_page_ids=False)
        raise pa.UnsupportedLayout("pages_per_iter must be a power of two >= 1")
    del allow_tf32, num_warps, num_stages
    if q.dim() == 4 and q.stride(-1) != 1:
        q = q.contiguous()
    key = _plan_key(q, kv, scale, num_splits, out, workspace, status)
    plan = _PLANS.get(key) if key is not None and not check_page_ids else None
    if plan is None:
        plan = DecodePlan(q, kv, scale, num_splits=num_splits, out=out, workspace=workspace,
                          status=status, check_page_ids=check_page_ids)
        if key is not None and out is not None and workspace is not None:
            if len(_PLANS) >= _PLAN_CACHE_SIZE:
                _PLANS.pop(next(iter(_PLANS)))
            _PLANS[key] = plan
    if q.device.index == torch.cuda.current_device():
        return plan.run()
    with torch.cuda.device(q.device):
        return plan.run()


_PREFILL_WS: dict = {}


@torch.no_grad()
def packed_prefill_attention(q: torch.Tensor, kv: pa.PackedKV, scale: float, *,
                             num_splits: int | None = None, check_page_ids: bool = True,
                             status: torch.Tensor | None = None,
                             workspace: torch.Tensor | None = None) -> torch.Tensor:
    """Causal attention of a chunk of Q query tokens per sequence over the
    packed pages (`wtq_prefill`): q (B, Hq, Q, D) -> (B, Hq, Q, D) in q.dtype,
    returned as a view of a (B, Q, Hq, D) tensor (the layout attention
    interfaces hand back).  The chunk's own K/V must already be appended:
    `kv.seq_lens` includes the Q tokens, and token i of the chunk sees keys
    [0, seq_len - Q + i].  The pages are read and decoded once for all query
    rows.  Raises `BackendError` (WTQ_ERR_UNSUPPORTED) for layouts only the
    row-by-row decode path serves; `prefill_supported()` asks first."""
    pa.check_contract(q, kv, check_page_ids=check_page_ids)
    if not q.is_cuda:
        raise pa.UnsupportedLayout("the CUDA prefill kernel needs CUDA tensors")
    B, Hq, Q, D = q.shape
    dev = q.device
    Hkv, S, P = kv.num_kv_heads, kv.page_size, kv.k_pages.shape[0]
    max_pages = kv.page_table.shape[1]
    out = torch.empty(B, Q, Hq, D, dtype=q.dtype, device=dev)
    if B == 0 or Q == 0:
        return out.permute(0, 2, 1, 3)
    if max_pages == 0:
        return out.zero_().permute(0, 2, 1, 3)
    rows = q.permute(0, 2, 1, 3).contiguous()                 # (B, Q, Hq, D): row b * Q + i
    L = _lib.lib()
    asked = max(int(num_splits or 0), 0)                      # 0: the library chooses the schedule
    splits = asked or L.wtq_prefill_auto_splits(B, Hq, Hkv, Q, max_pages, S)
    need = L.wtq_prefill_workspace_bytes(B, Hq, Hkv, Q, D, splits)
    if workspace is None:
        key = (dev.index, torch.cuda.current_stream(dev).cuda_stream)
        workspace = _PREFILL_WS.get(key)
        if workspace is None or workspace.numel() < need:
            workspace = _PREFILL_WS[key] = torch.empty(need, dtype=torch.uint8, device=dev)
    k_side = _side(kv.k_pages, kv.k_norms, kv.k_quant)
    v_side = _side(kv.v_pages, kv.v_norms, kv.v_quant)
    with torch.cuda.device(dev):
        _lib.check(L.wtq_prefill(
            rows.data_ptr(), _lib.dtype_code(q.dtype), _lib.i64x(Hq * D, D), out.data_ptr(),
            _lib.i64x(Hq * D, D), ctypes.byref(k_side), ctypes.byref(v_side),
            kv.page_table.data_ptr(), kv.page_table.stride(0), kv.seq_lens.data_ptr(), float(scale),
            B, Hq, Hkv, Q, D, S, P, max_pages, asked, workspace.data_ptr(), workspace.numel(),
            status.data_ptr() if status is not None else None,
            torch.cuda.current_stream(dev).cuda_stream))
    return out.permute(0, 2, 1, 3)


def prefill_supported(q: torch.Tensor, kv: pa.PackedKV) -> bool:
    """Whether `packed_prefill_attention` serves this layout (head_dim 128, a
    width pair with a tensor-core kernel, power-of-two pages of at least 16
    tokens, at most 8 query heads per kv head, 16-byte aligned pages)."""
    D, S = kv.head_dim, kv.page_size
    widths = (kv.k_quant.bit_width, kv.v_quant.bit_width)
    ok = (q.is_cuda and D == 128 and widths in ((4, 4), (4, 6), (6, 6), (8, 8)) and S >= 16
          and S & (S - 1) == 0 and q.shape[1] // kv.num_kv_heads <= 8
          and q.dtype in (torch.float32, torch.float16, torch.bfloat16))
    for pages, norms in ((kv.k_pages, kv.k_norms), (kv.v_pages, kv.v_norms)):
        ok = ok and pages.data_ptr() % 16 == 0 and norms.data_ptr() % 16 == 0 \
            and pages.stride(0) % 16 == 0 and pages.stride(1) % 16 == 0 \
            and norms.stride(0) % 8 == 0 and norms.stride(1) % 8 == 0 \
            and pages.stride(-1) == 1 and pages.stride(-2) == pages.shape[-1] and norms.stride(-1) == 1
    return bool(ok and kv.page_table.stride(-1) == 1 and kv.seq_lens.is_contiguous())


@torch.no_grad()
def dense_decode_attention(q: torch.Tensor, kv: "pa.DenseKV", scale: float, *, num_splits: int = 1,
                           allow_tf32: bool = False, num_warps: int = 4, num_stages: int = 2,
                           pages_per_iter: int = 1, status: torch.Tensor | None = None) -> torch.Tensor:
    """Unquantised paged decode with the same split-K schedule: the matched
    baseline arm (reference: turboquant_kv/packed_attention_triton.py:190-201).
    q (B, Hq, 1, D) -> (B, Hq, 1, D) in q.dtype; pages (P, Hkv, S, D) in fp16,
    bf16 or fp32.  `num_splits` <= 0 picks about four blocks per SM.  The
    Triton tuning keywords are accepted and ignored."""
    del allow_tf32, num_warps, num_stages, pages_per_iter
    if q.dim() != 4 or q.shape[2] != 1 or not q.is_cuda:
        raise pa.UnsupportedLayout("dense kernel: CUDA decode only (one query token per sequence)")
    B, Hq, _, D = q.shape
    kp, vp = kv.k_pages, kv.v_pages
    if (kp.dim() != 4 or kp.shape != vp.shape or kp.dtype != vp.dtype or kp.shape[3] != D
            or kp.stride(-1) != 1 or kp.stride(-2) != D or vp.stride(-1) != 1 or vp.stride(-2) != D
            or kp.dtype not in (torch.float32, torch.float16, torch.bfloat16) or D > 256):
        raise pa.UnsupportedLayout("dense kernel: unsupported page layout")
    Hkv, S, P = kp.shape[1], kp.shape[2], kp.shape[0]
    if Hq % Hkv or kv.page_table.dtype != torch.int32 or kv.seq_lens.dtype != torch.int32 \
            or kv.page_table.shape[0] != B or kv.page_table.stride(-1) != 1:
        raise pa.UnsupportedLayout("dense kernel: malformed page table, lengths or head counts")
    dev = _lib.require_cuda(q, kp, vp, kv.page_table, kv.seq_lens)
    if q.stride(-1) != 1:
        q = q.contiguous()
    out = torch.empty(B, Hq, 1, D, dtype=q.dtype, device=dev)
    max_pages = kv.page_table.shape[1]
    if B == 0 or max_pages == 0:
        return out.zero_()
    splits = int(num_splits or 0)
    if splits <= 0:
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        tiles = max(1, -(-max_pages * S // 32))
        splits = max(1, min(tiles, -(-4 * sms // max(B * Hkv, 1)), 1024))
    lib = _lib.lib()
    ws = torch.empty(lib.wtq_dense_workspace_bytes(B, Hq, D, splits), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.wtq_dense_decode(
            q.data_ptr(), _lib.dtype_code(q.dtype), _lib.i64x(q.stride(0), q.stride(1)),
            out.data_ptr(), _lib.i64x(out.stride(0), out.stride(1)), kp.data_ptr(), vp.data_ptr(),
            _lib.dtype_code(kp.dtype), _lib.i64x(kp.stride(0), kp.stride(1)),
            _lib.i64x(vp.stride(0), vp.stride(1)), kv.page_table.data_ptr(), kv.page_table.stride(0),
            kv.seq_lens.contiguous().data_ptr(), float(scale), B, Hq, Hkv, D, S, P, max_pages, splits,
            ws.data_ptr(), ws.numel(), status.data_ptr() if status is not None else None,
            _lib.stream_ptr(dev)))
    return out


# Serving loops call the operator every step with the same buffers (query and
# output staging tensors, one layer's pages, the batch's table and lengths,
# updated in place).  When the caller supplies `out` and `workspace` and has
# vouched for the page ids, the checked and marshalled call is remembered under
# the identity (address, shape, strides) of every tensor involved, so a repeat
# costs one dictionary lookup instead of the contract checks.  A plan keeps its
# tensors alive, so a remembered address cannot be reused by another tensor.
_PLANS: dict = {}
_PLAN_CACHE_SIZE = 256


def _ident(t: torch.Tensor):
    return (t.data_ptr(), tuple(t.shape), t.stride(), t.dtype)


def _plan_key(q, kv, scale, num_splits, out, workspace, status):
    try:
        return (_ident(q), _ident(kv.k_pages), _ident(kv.v_pages), _ident(kv.k_norms),
                _ident(kv.v_norms), _ident(kv.page_table), _ident(kv.seq_lens),
                kv.k_quant.Pi.data_ptr(), kv.k_quant.centroids.data_ptr(), kv.k_quant.bit_width,
                kv.v_quant.Pi.data_ptr(), kv.v_quant.centroids.data_ptr(), kv.v_quant.bit_width,
                kv.head_dim, float(scale), int(num_splits or 0),
                None if out is None else _ident(out),
                None if workspace is None else _ident(workspace),
                None if status is None else status.data_ptr())
    except Exception:                                  # noqa: BLE001 - malformed input: take the checked path
        return None
