"""GPU parity of packed decode attention: the CUDA path through the C ABI
against the reference's stored outputs and the CPU oracle on the same bytes.
Bounds: max-abs 2e-3 and relative L2 1e-3 (fp32 accumulation)."""
import numpy as np
import pytest
import torch

import cases
from helpers import ATOL, assert_attention_close, oracle_case, to_device
from oracle import tq_oracle as orc
from winnow_b200 import _lib, packed_attention as pa, packed_backend as pb, workloads
from winnow_b200.cache import _get_quantizer, dequantize_rows
from winnow_b200.packed_attention_cuda import packed_decode_attention

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(params=["auto_path", "generic_path"])
def kernel_path(request, monkeypatch):
    """Run a test once with the library's own kernel choice (the tensor-core
    kernel where the shape allows it) and once forced onto the generic kernels."""
    if request.param == "generic_path":
        monkeypatch.setenv("WTQ_FORCE_GENERIC", "1")
    else:
        monkeypatch.delenv("WTQ_FORCE_GENERIC", raising=False)
    return request.param


@pytest.mark.parametrize("splits", [None, 1, 3])
@pytest.mark.parametrize("c", cases.ATTENTION_CASES, ids=lambda c: c.name)
def test_decode_matches_reference(golden, c, splits, kernel_path):
    tensor_core = (c.D == 128 and (c.bw_k, c.bw_v) in ((4, 4), (4, 6), (6, 6), (8, 8))
                   and c.Hq // c.Hkv <= 8 and c.S >= 16 and c.S & (c.S - 1) == 0)
    if kernel_path == "generic_path" and not tensor_core:
        pytest.skip("this shape takes the generic kernels on the automatic path already")
    q, okv, _ = oracle_case(c)
    ref = torch.from_numpy(golden("attention")[f"{c.name}/out"])
    got = packed_decode_attention(q.to(DEV), to_device(okv, DEV), orc.default_scale(c.D),
                                  num_splits=splits)
    assert got.shape == q.shape and got.dtype == q.dtype
    assert_attention_close(got, ref)        # plain bounds: 2e-3 max-abs, 1e-3 relative L2
    for b, L in enumerate(c.lens):
        if L == 0:
            assert (got[b] == 0).all()


def test_config1_outputs(golden, kernel_path):
    g = golden("config1")
    w = workloads.WORKLOADS["config1"]
    q = workloads.queries(w)
    kq, vq = _get_quantizer(4, 128, DEV, 42), _get_quantizer(4, 128, DEV, 43)
    kv = pa.PackedKV(*(torch.from_numpy(g[n]).to(DEV) for n in ("k_pages", "k_norms", "v_pages", "v_norms")),
                     torch.from_numpy(g["page_table"]).to(DEV),
                     torch.tensor(w.seq_lens(), dtype=torch.int32, device=DEV),
                     pa.Quantizer.from_tq(kq), pa.Quantizer.from_tq(vq), 128)
    got = packed_decode_attention(q.to(DEV), kv, pa.default_scale(128))
    assert_attention_close(got, torch.from_numpy(g["out_tiled"]))
    assert_attention_close(got, torch.from_numpy(g["out_reconstruct"]))


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 2e-2), (torch.float16, 3e-3)])
def test_low_precision_query_dtype(dtype, tol):
    c = cases.AttnCase("lp", 3, 2, 28, 4, 128, (60, 9), 16, 8, 8)
    q, okv, _ = oracle_case(c)
    ql = q.to(dtype)
    got = packed_decode_attention(ql.to(DEV), to_device(okv, DEV), orc.default_scale(128))
    assert got.dtype == dtype
    ref = orc.tiled_attention(ql.float(), okv, orc.default_scale(128))
    assert (got.float().cpu() - ref).abs().max() < tol


def test_strided_pool_layer_view_and_output_slice():
    """One layer of a (layers, P, ...) pool, storage offset > 0, and the result
    written into a slice of a wider (B, Hq_total, 1, D) buffer."""
    c = cases.AttnCase("strided", 4, 2, 8, 2, 64, (45, 20), 16, 8, 8)
    q, okv, _ = oracle_case(c)
    kv = to_device(okv, DEV)
    mid = lambda t: torch.stack([torch.zeros_like(t), t, torch.zeros_like(t)])[1]
    kv2 = pa.PackedKV(mid(kv.k_pages), mid(kv.k_norms), mid(kv.v_pages), mid(kv.v_norms),
                      kv.page_table, kv.seq_lens, kv.k_quant, kv.v_quant, kv.head_dim)
    assert kv2.k_pages.storage_offset() > 0
    wide = torch.full((2, 24, 1, 64), 7.0, device=DEV)
    out = packed_decode_attention(q.to(DEV), kv2, orc.default_scale(64), out=wide[:, 8:16])
    ref = orc.tiled_attention(q, okv, orc.default_scale(64))
    assert_attention_close(out, ref)
    assert (wide[:, :8] == 7).all() and (wide[:, 16:] == 7).all()
    assert_attention_close(wide[:, 8:16], ref)


def test_rejects_before_launch():
    c = cases.AttnCase("rej", 5, 2, 8, 2, 64, (20, 3), 16, 8, 8)
    q, okv, _ = oracle_case(c)
    kv = to_device(okv, DEV)
    with pytest.raises(pa.UnsupportedLayout):
        packed_decode_attention(q.repeat(1, 1, 2, 1).to(DEV), kv, 1.0)            # Q = 2
    with pytest.raises(pa.UnsupportedLayout):
        packed_decode_attention(q.to(DEV), kv, 1.0, pages_per_iter=3)
    bad = pa.PackedKV(**{**kv.__dict__, "page_table": kv.page_table.clone()})
    bad.page_table[0, 0] = kv.k_pages.shape[0]
    with pytest.raises(pa.UnsupportedLayout):
        packed_decode_attention(q.to(DEV), bad, 1.0)
    # with the host check skipped the kernel itself refuses the id, flags it,
    # and treats the page as masked instead of reading it
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = packed_decode_attention(q.to(DEV), bad, 1.0, check_page_ids=False, status=status)
    assert int(status.item()) & _lib.STATUS_BAD_PAGE
    assert torch.isfinite(out).all()


def test_stale_slots_are_masked_not_trusted(kernel_path):
    """Slots past seq_len hold garbage from a recycled page; results must not change."""
    c = cases.AttnCase("stale", 9, 2, 8, 2, 128, (21, 5), 16, 4, 4)
    q, okv, _ = oracle_case(c)
    ref = orc.tiled_attention(q, okv, orc.default_scale(128))
    kv = to_device(okv, DEV)
    g = torch.Generator().manual_seed(1)
    for b, L in enumerate(c.lens):
        pid = int(okv.page_table[b, (L - 1) // 16])
        kv.k_pages[pid, :, L % 16:] = torch.randint(0, 255, kv.k_pages[pid, :, L % 16:].shape,
                                                    generator=g, dtype=torch.uint8).to(DEV)
        kv.v_norms[pid, :, L % 16:] = float("inf")
        kv.k_norms[pid, :, L % 16:] = 6e4
    assert_attention_close(packed_decode_attention(q.to(DEV), kv, orc.default_scale(128)), ref)


def test_workspace_is_independent_of_history_length():
    L = _lib.lib()
    a = L.wtq_decode_workspace_bytes(8, 28, 4, 128, 1024 // 32, 32, 4)
    b = L.wtq_decode_workspace_bytes(8, 28, 4, 128, 16384 // 32, 32, 4)
    assert a == b
    assert b < 8 * 4 * 16384 * 128 * 2 / 50


@pytest.mark.parametrize("bw", [4, 6, 8, 3])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_dequant_golden(golden, bw, dtype):
    g = golden("dequant")
    tq = _get_quantizer(bw, 128, DEV, 42)
    packed = torch.from_numpy(g[f"b{bw}/packed"]).to(DEV)
    norms = torch.from_numpy(g[f"b{bw}/norms"]).to(DEV)
    n = packed.shape[0]
    guard = torch.full((n + 64, 128), -12352.0, dtype=dtype, device=DEV)    # canary tail
    dequantize_rows(packed, norms, tq.centroids, tq.Pi, bw, 128, out=guard[:n])
    ref = torch.from_numpy(g[f"b{bw}/out_f32"])
    got = guard[:n].float().cpu()
    assert (guard[n:] == -12352.0).all()
    if dtype == torch.float32:
        assert torch.allclose(got, ref, rtol=1e-5, atol=1e-6 * float(ref.abs().max()))
    else:
        # At most one bf16 unit in the last place away from the rounded reference.
        # Outputs that cancel to almost nothing carry the fp32 summation noise of
        # the reference itself (its own value for the one such element of the
        # 8-bit fixture is 3% off the exactly summed one), so 1e-6 of the largest
        # output is allowed on top.
        rb = ref.to(torch.bfloat16).float()
        ulp = rb.abs() * 2.0 ** -7 + 1e-6 * float(ref.abs().max())
        assert ((got - rb).abs() <= ulp).all()


def test_dequant_strided_cache_slice():
    """(B, H, L, NB) view of a (B, H, MAXLEN, NB) buffer, read in place."""
    B, H, MAXLEN, L, bw = 2, 3, 40, 27, 4
    tq = _get_quantizer(bw, 128, DEV, 42)
    g = torch.Generator().manual_seed(4)
    buf = torch.randint(0, 256, (B, H, MAXLEN, 64), generator=g, dtype=torch.uint8)
    nbuf = (torch.rand(B, H, MAXLEN, generator=g) * 50).half()
    out = dequantize_rows(buf.to(DEV)[:, :, :L], nbuf.to(DEV)[:, :, :L], tq.centroids, tq.Pi, bw, 128,
                          out=torch.empty(B, H, L, 128, device=DEV))
    o = orc.OracleQuantizer.get(bw, 128, 42)
    ref = orc.dequantize_rows(buf[:, :, :L].contiguous(), nbuf[:, :, :L].contiguous(),
                              o.centroids, o.Pi, bw, 128)
    assert torch.allclose(out.cpu(), ref, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("bw", [4, 6, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("mode", ["tc", "tc_fast", "tc_mma", "tc_fast_mma"])
def test_dequant_tensor_core_modes(bw, dtype, mode):
    """Tensor-core dequantisation against the oracle on rows that end inside a
    32-row tile and planes (L = 27 of MAXLEN = 40) that end inside one: "tc"
    (split operands) must sit within one unit in the last place of the rounded
    oracle value for 16-bit outputs and within fp32 rounding for fp32; "tc_fast"
    (single fp16 operands) is held to the error of fp16-rounded operands, 2^-9
    of the largest output."""
    B, H, MAXLEN, L = 2, 3, 40, 27
    nb = 16 * bw
    tq = _get_quantizer(bw, 128, DEV, 42)
    g = torch.Generator().manual_seed(40 + bw)
    buf = torch.randint(0, 256, (B, H, MAXLEN, nb), generator=g, dtype=torch.uint8)
    nbuf = (torch.rand(B, H, MAXLEN, generator=g) * 50 + 0.5).half()
    guard = torch.full((B * H * L + 40, 128), -12352.0, dtype=dtype, device=DEV)
    out = guard[:B * H * L].view(B, H, L, 128)
    dequantize_rows(buf.to(DEV)[:, :, :L], nbuf.to(DEV)[:, :, :L], tq.centroids, tq.Pi, bw, 128,
                    out=out, mode=mode)
    assert (guard[B * H * L:] == -12352.0).all()
    o = orc.OracleQuantizer.get(bw, 128, 42)
    ref = orc.dequantize_rows(buf[:, :, :L].contiguous(), nbuf[:, :, :L].contiguous(),
                              o.centroids, o.Pi, bw, 128)
    got = out.float().cpu()
    top = float(ref.abs().max())
    if mode.startswith("tc_fast"):
        assert float((got - ref).abs().max()) <= 2.0 ** -9 * top + (0 if dtype == torch.float32 else 2.0 ** -8 * top)
        return
    if dtype == torch.float32:
        assert float((got - ref).abs().max()) <= 4e-6 * top
    else:
        eps = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10
        rounded = ref.to(dtype).float()
        # one unit in the last place, plus the split's own error for outputs that
        # cancel to almost nothing
        assert ((got - rounded).abs() <= rounded.abs() * eps + 4e-6 * top).all()


def test_dequant_tensor_core_refuses_what_it_cannot_do():
    tq = _get_quantizer(4, 64, DEV, 42)
    packed = torch.zeros(8, 32, dtype=torch.uint8, device=DEV)
    norms = torch.ones(8, dtype=torch.float16, device=DEV)
    with pytest.raises(_lib.BackendError, match="head_dim must be 128"):
        dequantize_rows(packed, norms, tq.centroids, tq.Pi, 4, 64, mode="tc")
    out = dequantize_rows(packed, norms, tq.centroids, tq.Pi, 4, 64, allow_tf32=True)   # falls to exact
    assert out.shape == (8, 64)


def test_attention_interface_entry_point():
    """winnow_packed_attention: decode goes to the CUDA operator, a prefill
    chunk to dequantize + SDPA; both agree with the oracle."""
    c = cases.AttnCase("iface", 21, 2, 8, 2, 128, (40, 17), 16, 4, 4)
    k, v, q, g = cases.attention_inputs(c)
    okv = orc.pages_from_dense(k, v, c.lens, orc.OracleQuantizer.get(4, 128, 42),
                               orc.OracleQuantizer.get(4, 128, 43), 16, generator=g)
    kv = to_device(okv, DEV)
    pb.BACKEND_COUNTS.clear()
    out, _ = pb.winnow_packed_attention(None, q.to(DEV), kv, kv, None, scaling=0.09)
    assert out.shape == (2, 1, 8, 128) and pb.BACKEND_COUNTS["cuda_packed"] == 1
    assert_attention_close(out.transpose(1, 2), orc.tiled_attention(q, okv, 0.09))
    kv.decode_backend = "triton_packed"
    pb.winnow_packed_attention(None, q.to(DEV), kv, kv, None, scaling=0.09)
    assert pb.BACKEND_COUNTS["cuda_packed"] == 2 and pb.BACKEND_COUNTS["triton_packed"] == 1
    gq = torch.Generator().manual_seed(5)
    q5 = torch.randn(2, 8, 5, 128, generator=gq)
    out5, _ = pb.winnow_packed_attention(None, q5.to(DEV), kv, kv, None, scaling=0.09)
    assert pb.BACKEND_COUNTS["prefill_reconstruct_sdpa"] == 1      # a bare handle: the reference's path
    ref5 = orc.reconstruct_attention(q5, okv, 0.09)
    assert (out5.transpose(1, 2).cpu() - ref5).abs().max() < 2e-3
    kv.prefill_backend = "packed"        # additive: the chunk on the page-scan kernels
    out5p, _ = pb.winnow_packed_attention(None, q5.to(DEV), kv, kv, None, scaling=0.09)
    assert pb.BACKEND_COUNTS["prefill_cuda_packed"] == 1
    assert out5p.shape == out5.shape and out5p.dtype == out5.dtype
    assert (out5p.transpose(1, 2).cpu() - ref5).abs().max() < 2e-3


def test_append_then_decode_through_the_cache():
    """One engine-style step: reserve pages, update() every layer, attend."""
    from winnow_b200.page_pool import PagePool
    B, Hq, Hkv, D, S = 3, 8, 2, 128, 16
    lens = (33, 0, 16)
    kq, vq = _get_quantizer(4, D, DEV, 42), _get_quantizer(6, D, DEV, 43)
    oq, ov = orc.OracleQuantizer.get(4, D, 42), orc.OracleQuantizer.get(6, D, 43)
    pool = PagePool(num_layers=1, num_pages=12, num_kv_heads=Hkv, page_size=S, nb_k=64, nb_v=96,
                    device=DEV)
    owners = ["a", "b", "c"]
    g = torch.Generator().manual_seed(77)
    hist_k = torch.randn(B, Hkv, 40, D, generator=g)
    hist_v = torch.randn(B, Hkv, 40, D, generator=g)
    # prefill each sequence alone (n = its length), then one batched decode step
    for b, (o, L) in enumerate(zip(owners, lens)):
        pool.ensure(o, L + 1)
        if L:
            cache = pb.PagedPackedCache(pool, [o], [0], k_quant=kq, v_quant=vq, head_dim=D)
            cache.update(hist_k[b:b + 1, :, :L].to(DEV), hist_v[b:b + 1, :, :L].to(DEV), 0)
    cache = pb.PagedPackedCache(pool, owners, list(lens), k_quant=kq, v_quant=vq, head_dim=D)
    new_k = torch.randn(B, Hkv, 1, D, generator=g)
    new_v = torch.randn(B, Hkv, 1, D, generator=g)
    handle, _ = cache.update(new_k.to(DEV), new_v.to(DEV), 0)
    q = torch.randn(B, Hq, 1, D, generator=g)
    out, _ = pb.winnow_packed_attention(None, q.to(DEV), handle, handle, None)
    # oracle: same pool layout, filled by the oracle's append
    table = handle.page_table.cpu()
    kp = torch.zeros(12, Hkv, S, 64, dtype=torch.uint8); vp = torch.zeros(12, Hkv, S, 96, dtype=torch.uint8)
    kn = torch.zeros(12, Hkv, S, dtype=torch.float16); vn = torch.zeros(12, Hkv, S, dtype=torch.float16)
    for b, L in enumerate(lens):
        if L:
            orc.append_tokens(kp, kn, vp, vn, table[b:b + 1], [0], hist_k[b:b + 1, :, :L],
                              hist_v[b:b + 1, :, :L], oq, ov)
    orc.append_tokens(kp, kn, vp, vn, table, lens, new_k, new_v, oq, ov)
    assert torch.equal(pool.k_pages[0].cpu(), kp) and torch.equal(pool.v_pages[0].cpu(), vp)
    assert torch.equal(pool.k_norms[0].cpu(), kn) and torch.equal(pool.v_norms[0].cpu(), vn)
    okv = orc.OracleKV(kp, kn, vp, vn, table, torch.tensor([L + 1 for L in lens], dtype=torch.int32),
                       oq.Pi, oq.centroids, 4, ov.Pi, ov.centroids, 6, D)
    assert_attention_close(out.transpose(1, 2), orc.tiled_attention(q, okv, D ** -0.5))


def test_repeated_calls_reuse_the_marshalled_plan():
    """Same buffers, page ids vouched for: the second call takes the remembered
    plan, sees data updated in place, and still matches the oracle."""
    from winnow_b200 import packed_attention_cuda as pac
    c = cases.AttnCase("plan", 31, 2, 8, 2, 128, (70, 33), 16, 4, 4)
    q, okv, _ = oracle_case(c)
    kv = to_device(okv, DEV)
    scale = orc.default_scale(128)
    qd = q.to(DEV)
    out = torch.empty_like(qd)
    ws = pac.decode_workspace(2, 8, 2, 128, kv.page_table.shape[1], 16, 0, DEV)
    pac._PLANS.clear()
    first = packed_decode_attention(qd, kv, scale, out=out, workspace=ws, check_page_ids=False).clone()
    assert len(pac._PLANS) == 1
    q2 = torch.randn(q.shape, generator=torch.Generator().manual_seed(5))
    qd.copy_(q2)                                         # new query, same buffer
    second = packed_decode_attention(qd, kv, scale, out=out, workspace=ws, check_page_ids=False)
    assert len(pac._PLANS) == 1 and second.data_ptr() == out.data_ptr()
    assert_attention_close(first, orc.tiled_attention(q, okv, scale))
    assert_attention_close(second, orc.tiled_attention(q2, okv, scale))
    # a checked call never uses the cache
    packed_decode_attention(qd, kv, scale, out=out, workspace=ws)
    assert len(pac._PLANS) == 1


def test_legacy_contiguous_cache_roundtrip():
    """TQPackedLayer: write in place, dequantize the history; against the oracle."""
    from winnow_b200.cache import TQPackedCache
    g = torch.Generator().manual_seed(12)
    B, H, D, bw = 2, 3, 128, 4
    cache = TQPackedCache(D, bw, DEV, max_cache_len=64, num_layers=2)
    o = orc.OracleQuantizer.get(bw, D, 42)
    hist_k, hist_v = [], []
    for n in (17, 1, 1):                               # a prefill chunk, then two decode steps
        k = torch.randn(B, H, n, D, generator=g).to(torch.bfloat16)
        v = torch.randn(B, H, n, D, generator=g).to(torch.bfloat16)
        hist_k.append(k), hist_v.append(v)
        K, V = cache.update(k.to(DEV), v.to(DEV), 1)
    assert cache.get_seq_length(1) == 19 and K.shape == (B, H, 19, D) and K.dtype == torch.bfloat16
    for dense, got in ((torch.cat(hist_k, 2), K), (torch.cat(hist_v, 2), V)):
        # same call grouping as the cache's three updates
        parts = []
        for chunk in dense.split([17, 1, 1], dim=2):
            idx, nrm = o.quantize(chunk)
            parts.append(orc.dequantize_rows(orc.pack(idx, bw), nrm.to(torch.float16),
                                             o.centroids, o.Pi, bw, D))
        ref = torch.cat(parts, 2).to(torch.bfloat16).float()
        ulp = (ref.abs() * 2.0 ** -7).clamp(min=1e-30)
        assert ((got.float().cpu() - ref).abs() <= ulp).all()
    assert cache.layers[1].last_dispatch_decision.backend == "cuda_sm100"
    with pytest.raises(RuntimeError):
        cache.update(torch.zeros(B, H, 64, D, device=DEV), torch.zeros(B, H, 64, D, device=DEV), 1)


def test_legacy_cache_outlier_channels_and_hf_protocol():
    """The 3.5-bit operating point of the reference's legacy cache
    (turboquant_kv/cache.py:183-191,224-233,289-303): 32 outlier channels at 4
    bits, the other 96 at 3 bits, each part with its own rotation, codebook and
    norms.  Checked against the oracle's quantizers applied to the same channel
    split; the classes are `transformers` cache classes and keep the
    reference's accounting helpers."""
    from transformers.cache_utils import DynamicCache, DynamicLayer
    from winnow_b200.cache import TQPackedCache, TQPackedLayer
    from winnow_b200.native_kernel import existing_native_kernel
    assert issubclass(TQPackedCache, DynamicCache) and issubclass(TQPackedLayer, DynamicLayer)
    g = torch.Generator().manual_seed(31)
    B, H, D, n_out = 2, 2, 128, 32
    cache = TQPackedCache(D, 3, DEV, max_cache_len=40, num_layers=1,
                          num_outlier_channels=n_out, outlier_bits=4)
    boost = torch.ones(D)
    boost[torch.randperm(D, generator=g)[:n_out]] = 6.0          # clear outlier channels
    chunks_k, chunks_v = [], []
    for n in (9, 1):
        k = (torch.randn(B, H, n, D, generator=g) * boost).to(torch.bfloat16)
        v = (torch.randn(B, H, n, D, generator=g) * boost).to(torch.bfloat16)
        chunks_k.append(k), chunks_v.append(v)
        K, V = cache.update(k.to(DEV), v.to(DEV), 0)
    layer = cache.layers[0]
    assert K.shape == (B, H, 10, D) and cache.get_seq_length() == 10
    assert layer.get_mask_sizes(1) == (10, 0) and layer.get_max_cache_shape() == 40
    rms = chunks_k[0].float().pow(2).mean(dim=(0, 1, 2)).sqrt()
    mask = torch.zeros(D, dtype=torch.bool)
    mask[rms.topk(n_out).indices] = True
    assert torch.equal(layer._mask.cpu(), mask)
    reg, out = orc.OracleQuantizer.get(3, D - n_out, 42), orc.OracleQuantizer.get(4, n_out, 43)
    for chunks, got in ((chunks_k, K), (chunks_v, V)):
        ref = torch.zeros(B, H, 10, D)
        at = 0
        for chunk in chunks:                                    # same call grouping as the updates
            n = chunk.shape[2]
            for o, sel, bw, dim in ((reg, ~mask, 3, D - n_out), (out, mask, 4, n_out)):
                idx, nrm = o.quantize(chunk.float()[..., sel])
                part = orc.dequantize_rows(orc.pack(idx, bw), nrm.to(torch.float16),
                                           o.centroids, o.Pi, bw, dim)
                ref[:, :, at:at + n][..., sel] = part
            at += n
        ref = ref.to(torch.bfloat16).float()
        ulp = (ref.abs() * 2.0 ** -7).clamp(min=1e-30)
        assert ((got.float().cpu() - ref).abs() <= ulp).all()
    assert abs(cache.effective_bits() - 3.5) < 1e-9
    assert cache.persistent_bytes() == 2 * B * H * 40 * (36 + 16 + 4)
    assert cache.persistent_bytes_used() == cache.persistent_bytes() * 10 // 40
    assert cache.transient_bytes() == 2 * B * H * 10 * D * 2
    layer.reset()
    assert cache.get_seq_length() == 0
    # the reference's adapter name for its native kernel resolves to wtq_dequant
    fn = existing_native_kernel()
    tq = _get_quantizer(4, 128, DEV, 42)
    packed = torch.randint(0, 256, (5, 64), dtype=torch.uint8, generator=g).to(DEV)
    norms = torch.rand(5, generator=g).half().to(DEV)
    a = fn(packed, norms, tq.centroids, tq.Pi, 4, 128, out=torch.empty(5, 128, device=DEV))
    b = dequantize_rows(packed, norms, tq.centroids, tq.Pi, 4, 128, out=torch.empty(5, 128, device=DEV))
    assert torch.equal(a, b)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("splits", [1, 3, 0])
def test_dense_page_arm_matches_sdpa(dtype, splits):
    """The unquantised paged arm (reference: turboquant_kv/test_packed_attention_triton.py:
    153-173): same page table walk, no codebook; against fp32 attention over the
    gathered history.  Also through the attention-interface entry point, under
    its own backend name and the reference's alias."""
    from winnow_b200.packed_attention_cuda import dense_decode_attention
    g = torch.Generator().manual_seed(9)
    B, Hq, Hkv, D, S = 3, 28, 4, 128, 16
    lens = (70, 0, 33)
    pages_n = sum(-(-L // S) for L in lens) + 2
    order = torch.randperm(pages_n, generator=g)
    kp = torch.randn(pages_n, Hkv, S, D, generator=g).to(dtype)
    vp = torch.randn(pages_n, Hkv, S, D, generator=g).to(dtype)
    table = torch.full((B, 6), -1, dtype=torch.int32)
    at = 0
    for b, L in enumerate(lens):
        n = -(-L // S)
        table[b, :n] = order[at:at + n].to(torch.int32)
        at += n
    q = (torch.randn(B, Hq, 1, D, generator=g) * 0.3).to(dtype)
    scale = D ** -0.5
    ref = torch.zeros(B, Hq, 1, D)
    for b, L in enumerate(lens):
        if L == 0:
            continue
        ids = table[b, : -(-L // S)].long()
        k = kp[ids].permute(1, 0, 2, 3).reshape(Hkv, -1, D)[:, :L].float().repeat_interleave(Hq // Hkv, 0)
        v = vp[ids].permute(1, 0, 2, 3).reshape(Hkv, -1, D)[:, :L].float().repeat_interleave(Hq // Hkv, 0)
        w = torch.softmax((q[b].float() @ k.transpose(1, 2)) * scale, dim=-1)
        ref[b] = w @ v
    kv = pa.DenseKV(kp.to(DEV), vp.to(DEV), table.to(DEV),
                    torch.tensor(lens, dtype=torch.int32, device=DEV), D)
    got = dense_decode_attention(q.to(DEV), kv, scale, num_splits=splits)
    assert got.dtype == dtype and got.shape == q.shape
    tol = 2e-2 if dtype == torch.bfloat16 else 2e-3
    assert (got.float().cpu() - ref).abs().max() < tol
    assert (got[1] == 0).all()
    pb.BACKEND_COUNTS.clear()
    out, _ = pb.winnow_packed_attention(None, q.to(DEV), kv, kv, None, scaling=scale)
    assert pb.BACKEND_COUNTS["cuda_dense"] == 1
    assert (out.transpose(1, 2).float().cpu() - ref).abs().max() < tol
    kv.decode_backend = "triton_dense"
    pb.winnow_packed_attention(None, q.to(DEV), kv, kv, None, scaling=scale)
    assert pb.BACKEND_COUNTS["cuda_dense"] == 2 and pb.BACKEND_COUNTS["triton_dense"] == 1
    with pytest.raises(pa.UnsupportedLayout):
        dense_decode_attention(q.repeat(1, 1, 2, 1).to(DEV), kv, scale)


def test_more_sequences_than_the_shared_prefix_holds():
    """1100 short ragged sequences: the chunk prefix no longer fits the kernel's
    shared-memory copy, so the work queue reads the one in the workspace."""
    g = torch.Generator().manual_seed(77)
    lens = tuple(int(x) for x in torch.randint(0, 41, (1100,), generator=g))
    c = cases.AttnCase("many", 78, len(lens), 2, 1, 128, lens, 16, 4, 4)
    q, okv, _ = oracle_case(c)
    got = packed_decode_attention(q.to(DEV), to_device(okv, DEV), orc.default_scale(128))
    assert_attention_close(got, orc.tiled_attention(q, okv, orc.default_scale(128)))
    for b, L in enumerate(lens):
        if L == 0:
            assert (got[b] == 0).all()


# 160 sequences x 4 kv heads per rank: enough groups for the small-block merge kernel
MANY_GROUPS = cases.AttnCase("many_groups", 3001, 160, 32, 8, 128,
                             tuple(1 + (37 * i) % 90 for i in range(160)), 16, 4, 4)


@pytest.mark.parametrize("name", ["val_long", "val_edges", "mixed_4k_6v", "many_groups"])
def test_exchange_epilogue_with_two_ranks_on_one_gpu(name):
    """`wtq_decode_exchange` for two ranks whose buffers both live on this GPU:
    the ranks' calls run one after the other on one stream (so no kernel ever
    waits for a kernel that has not been launched), each stores its head rows
    into both ranks' buffers and publishes its step; after both, each rank's
    bounded wait finds every flag set and both buffers hold the full output."""
    import ctypes
    from winnow_b200 import _lib, tp
    from winnow_b200.packed_attention_cuda import DecodePlan
    c = MANY_GROUPS if name == "many_groups" else next(
        (x for x in cases.ATTENTION_CASES if x.name == name), None)
    if c is None or c.Hkv % 2:
        pytest.skip("case not present or kv heads do not split in two")
    q, okv, _ = oracle_case(c)
    scale = orc.default_scale(c.D)
    dev = torch.device("cuda", 0)
    kv = to_device(okv, dev)
    world, B, D = 2, q.shape[0], c.D
    el = q.element_size()
    bufs = [[torch.zeros(B, c.Hq, 1, D, dtype=q.dtype, device=dev) for _ in range(2)]
            for _ in range(world)]                      # [rank][parity]
    flags = [torch.zeros(world, dtype=torch.int32, device=dev) for _ in range(world)]
    peer_out = [torch.tensor([bufs[r][i].data_ptr() for r in range(world)], dtype=torch.int64,
                             device=dev) for i in range(2)]
    peer_flags = torch.tensor([f.data_ptr() for f in flags], dtype=torch.int64, device=dev)
    lib = _lib.lib()
    ranks = []
    for rank in range(world):
        qs, ks = tp.head_shard(rank, world, c.Hq, c.Hkv)
        shard = pa.PackedKV(kv.k_pages[:, ks].contiguous(), kv.k_norms[:, ks].contiguous(),
                            kv.v_pages[:, ks].contiguous(), kv.v_norms[:, ks].contiguous(),
                            kv.page_table, kv.seq_lens, kv.k_quant, kv.v_quant, kv.head_dim)
        q_local = q[:, qs].contiguous().to(dev)
        hq = q_local.shape[1]
        plan = DecodePlan(q_local, shard, scale, out=bufs[rank][0][:, :hq])
        try:
            plan.run_exchange(None, dry_run=True)
        except _lib.BackendError:
            pytest.skip("shape has no exchange epilogue")
        ex = _lib.Exchange()
        ex.peer_out[0], ex.peer_out[1] = peer_out[0].data_ptr(), peer_out[1].data_ptr()
        ex.peer_flags = peer_flags.data_ptr()
        ex.out_strides[0], ex.out_strides[1] = bufs[0][0].stride(0), bufs[0][0].stride(1)
        ex.rank, ex.world, ex.head_offset = rank, world, rank * hq
        step = torch.zeros(4, dtype=torch.int32, device=dev)     # calls, waits, blocks per call
        done = torch.zeros(1, dtype=torch.int32, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        ex.step_counter, ex.done_counter = step.data_ptr(), done.data_ptr()
        ranks.append((plan, ex, step, done, status, q_local, qs))
    stream = torch.cuda.current_stream(dev).cuda_stream
    for call in (1, 2, 3):                               # parity 1, 0, 1 of the double buffer
        qi = q * (1.0 + 0.5 * (call - 1))
        for plan, ex, *_rest, q_local, qs in ranks:
            q_local.copy_(qi[:, qs])
            plan.run_exchange(ex)
        for rank, (plan, ex, step, done, status, *_r) in enumerate(ranks):
            _lib.check(lib.wtq_exchange_wait(flags[rank].data_ptr(), world, step.data_ptr(),
                                             1000, status.data_ptr(), stream))
        torch.cuda.synchronize()
        ref = orc.tiled_attention(qi, okv, scale)
        for rank, (plan, ex, step, done, status, *_r) in enumerate(ranks):
            assert int(status.item()) == 0
            calls, waits, blocks = step.tolist()[:3]
            assert calls == call and waits == call and blocks == 1 and int(done.item()) == 0
            assert flags[rank].tolist() == [call * blocks] * world
            assert_attention_close(bufs[rank][call & 1].float().cpu(), ref)


@pytest.mark.parametrize("name", ["val_tail", "mixed_4k_6v", "qwen7b_gqa_mixed", "gqa8_2"])
@pytest.mark.parametrize("Q", [1, 5])
def test_reference_operator_names_on_the_gpu(name, Q):
    """`tiled_compressed_attention`, `explicit_compressed_attention` and
    `reconstruct_attention` keep the reference's names, signatures and fp32
    result; a chunk of Q query tokens is causal inside the chunk (query i sees
    the keys up to its own position).  Checked against the CPU oracle."""
    c = next(x for x in cases.ATTENTION_CASES if x.name == name)
    q1, okv, _ = oracle_case(c)
    g = torch.Generator().manual_seed(c.seed + 17)
    q = torch.randn(q1.shape[0], q1.shape[1], Q, q1.shape[3], generator=g).to(q1.dtype)
    q = q * float(q1.float().std())
    scale = orc.default_scale(c.D)
    ref = orc.tiled_attention(q, okv, scale)
    assert ref.shape == q.shape
    dev = torch.device("cuda", 0)
    kv = to_device(okv, dev)
    qd = q.to(dev)
    for fn, kwargs in ((pa.tiled_compressed_attention, {}),
                       (pa.tiled_compressed_attention, {"split_pages": 3}),
                       (pa.explicit_compressed_attention, {}),
                       (pa.reconstruct_attention, {})):
        got = fn(qd, kv, scale, **kwargs)
        assert got.dtype == torch.float32 and got.shape == q.shape
        assert_attention_close(got.cpu(), ref)
    # rows of a chunk that reach before the start of a short sequence see nothing
    if Q > 1:
        lens = okv.seq_lens.tolist()
        got = pa.tiled_compressed_attention(qd, kv, scale).cpu()
        for b, L in enumerate(lens):
            for i in range(Q):
                if L - (Q - 1 - i) <= 0:
                    assert float(got[b, :, i].abs().max()) == 0.0


def test_exchange_wait_gives_up_and_says_so():
    """The bounded wait of the output exchange, made to run out on purpose: the
    arrival counts are short of what the call waits for (nothing will ever add
    to them), the poll limit is small, so the kernel must return, set
    WTQ_STATUS_EXCHANGE_TIMEOUT and leave the device usable; with the counts in
    place a later wait reports nothing."""
    lib = _lib.lib()
    dev = torch.device("cuda", 0)
    world, blocks = 2, 3
    flags = torch.zeros(world, dtype=torch.int32, device=dev)
    state = torch.tensor([0, 0, blocks, 0], dtype=torch.int32, device=dev)   # calls, waits, blocks
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream

    def wait():
        status.zero_()
        _lib.check(lib.wtq_exchange_wait(flags.data_ptr(), world, state.data_ptr(), 8,
                                         status.data_ptr(), stream))
        torch.cuda.synchronize()
        return int(status.item())

    assert wait() & _lib.STATUS_EXCHANGE_TIMEOUT            # wait 1: nobody arrived
    flags[0] = 2 * blocks                                    # wait 2: one rank complete, one short
    flags[1] = 2 * blocks - 1
    assert wait() & _lib.STATUS_EXCHANGE_TIMEOUT
    flags.fill_(3 * blocks)                                  # wait 3: everybody arrived
    assert wait() == 0
    assert state.tolist()[1] == 3
    assert float((torch.ones(4, device=dev) * 2).sum().item()) == 8.0   # the context still works
    # the merge blocks of the local call not recorded yet: that is "not arrived" too
    state[2] = 0
    assert wait() & _lib.STATUS_EXCHANGE_TIMEOUT
    # malformed calls are refused before any launch
    assert lib.wtq_exchange_wait(flags.data_ptr(), world, state.data_ptr(), 0, status.data_ptr(),
                                 stream) != 0
    assert lib.wtq_exchange_wait(None, world, state.data_ptr(), 8, status.data_ptr(), stream) != 0


# Seeded wrong implementations of the operator (the reference keeps the same
# list for its own suite, turboquant_kv/test_packed_attention.py:207-264): each
# is applied to the CPU oracle and must land at least 100 x ATOL away from what
# the GPU computes, i.e. the parity bound used throughout this file would
# notice that specific mistake if the kernels made it.
def _mutant_outputs(q, okv, scale):
    import copy
    D = okv.head_dim
    out = {}

    def run(kv=okv, qq=q, sc=scale, **kw):
        return orc.tiled_attention(qq, kv, sc, **kw)

    swapped = copy.copy(okv)                                   # q rotated with Pi instead of Pi^T
    swapped.k_Pi = okv.k_Pi.t().contiguous()
    out["transposed_query_rotation"] = run(kv=swapped)
    swapped = copy.copy(okv)                                   # output rotated with Pi^T
    swapped.v_Pi = okv.v_Pi.t().contiguous()
    out["transposed_output_rotation"] = run(kv=swapped)
    out["missing_scale"] = run(sc=1.0)
    wrong_basis = copy.copy(okv)                               # V decoded in the K basis
    wrong_basis.v_Pi = okv.k_Pi
    out["values_in_key_basis"] = run(kv=wrong_basis)
    Hq, Hkv = q.shape[1], okv.k_pages.shape[1]
    n_rep = Hq // Hkv
    if n_rep > 1 and Hkv > 1:                                  # h % Hkv head map instead of h // n_rep
        # head h must end up reading kv head h % Hkv: feed it to the oracle as head
        # (h % Hkv) * n_rep + h // Hkv, whose kv head under the right map is h % Hkv
        perm = torch.tensor([(h % Hkv) * n_rep + h // Hkv for h in range(Hq)])
        out["modulo_head_map"] = run(qq=q[:, torch.argsort(perm)])[:, perm]
    return out


@pytest.mark.parametrize("name", ["qwen7b_gqa_mixed", "gqa8_2", "val_long"])
def test_seeded_mutants_of_the_oracle_miss_the_gpu_output(name):
    c = next(x for x in cases.ATTENTION_CASES if x.name == name)
    q, okv, _ = oracle_case(c)
    scale = orc.default_scale(c.D)
    got = packed_decode_attention(q.to(DEV), to_device(okv, DEV), scale).float().cpu()
    assert_attention_close(got, orc.tiled_attention(q, okv, scale))
    mutants = _mutant_outputs(q, okv, scale)
    assert len(mutants) >= 4
    for label, wrong in mutants.items():
        miss = float((wrong - got).abs().max())
        assert miss >= 100 * ATOL, f"mutant {label} is only {miss:.3e} away from the GPU output"


@pytest.mark.parametrize("name", ["huge_scores", "val_huge"])
def test_online_softmax_mutants_miss_the_gpu_output(name):
    """The two schedule mutants of the reference's list, planted in the oracle:
    an online softmax that forgets to rescale its state when the maximum moves,
    and a split merge that adds chunk states without their weights.  Run on the
    cases whose scores are large enough for the maximum to move a lot."""
    c = next(x for x in cases.ATTENTION_CASES if x.name == name)
    q, okv, _ = oracle_case(c)
    scale = orc.default_scale(c.D)
    got = packed_decode_attention(q.to(DEV), to_device(okv, DEV), scale).float().cpu()
    assert_attention_close(got, orc.tiled_attention(q, okv, scale))
    for label, kwargs in (("update_without_rescale", {}), ("merge_without_rescale", {"split_pages": 1})):
        wrong = orc.tiled_attention(q, okv, scale, mutant=label, **kwargs)
        miss = float((wrong - got).abs().max())
        assert miss >= 100 * ATOL, f"mutant {label} is only {miss:.3e} away from the GPU output"
