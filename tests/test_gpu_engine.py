"""A decode loop on the device-resident step object: three layers, three
sequences of different lengths (one crosses a page boundary on the way), several
steps, with and without the captured graphs; pool bytes against the oracle's
append and attention outputs against its operator, layer by layer."""
import pytest
import torch

from helpers import assert_attention_close
from oracle import tq_oracle as orc
from winnow_b200 import packed_backend as pb
from winnow_b200.cache import _get_quantizer
from winnow_b200.engine_step import DecodeSession
from winnow_b200.page_pool import PagePool, StalePage

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0) if torch.cuda.is_available() else None


@pytest.mark.parametrize("graphs", [False, True])
def test_decode_session_matches_the_oracle_step_by_step(graphs):
    layers, B, Hq, Hkv, D, S = 3, 3, 8, 2, 128, 16
    start = (30, 0, 15)                                    # third sequence fills its page at once
    kq, vq = _get_quantizer(4, D, DEV, 42), _get_quantizer(6, D, DEV, 43)
    oq, ov = orc.OracleQuantizer.get(4, D, 42), orc.OracleQuantizer.get(6, D, 43)
    pool = PagePool(num_layers=layers, num_pages=16, num_kv_heads=Hkv, page_size=S, nb_k=64, nb_v=96,
                    device=DEV)
    owners = ["a", "b", "c"]
    g = torch.Generator().manual_seed(5)
    # history: written through the per-forward cache object, one sequence at a time
    hist = {}
    for b, (o, L) in enumerate(zip(owners, start)):
        pool.ensure(o, max(L, 1))
        if L:
            cache = pb.PagedPackedCache(pool, [o], [0], k_quant=kq, v_quant=vq, head_dim=D)
            for layer in range(layers):
                k = torch.randn(1, Hkv, L, D, generator=g)
                v = torch.randn(1, Hkv, L, D, generator=g)
                hist[(b, layer)] = (k, v)
                cache.update(k.to(DEV), v.to(DEV), layer)
            cache.check()
    sess = DecodeSession(pool, owners, start, k_quant=kq, v_quant=vq, head_dim=D, q_heads=Hq,
                         dtype=torch.float32, max_tokens=64)
    # the oracle's copy of the pool, filled the same way
    P = 16
    okp = [torch.zeros(P, Hkv, S, 64, dtype=torch.uint8) for _ in range(layers)]
    ovp = [torch.zeros(P, Hkv, S, 96, dtype=torch.uint8) for _ in range(layers)]
    okn = [torch.zeros(P, Hkv, S, dtype=torch.float16) for _ in range(layers)]
    ovn = [torch.zeros(P, Hkv, S, dtype=torch.float16) for _ in range(layers)]
    table0 = sess.table.table.cpu()
    for (b, layer), (k, v) in hist.items():
        orc.append_tokens(okp[layer], okn[layer], ovp[layer], ovn[layer], table0[b:b + 1], [0], k, v, oq, ov)
    lens = list(start)
    for step in range(4):
        sess.begin_step()
        if graphs and step == 1:
            sess.capture()
        table = sess.table.table.cpu()
        for layer in range(layers):
            k = torch.randn(B, Hkv, 1, D, generator=g)
            v = torch.randn(B, Hkv, 1, D, generator=g)
            q = torch.randn(B, Hq, 1, D, generator=g)
            out = sess.layer(layer, k.to(DEV), v.to(DEV), q.to(DEV)).clone()
            orc.append_tokens(okp[layer], okn[layer], ovp[layer], ovn[layer], table, lens, k, v, oq, ov)
            okv = orc.OracleKV(okp[layer], okn[layer], ovp[layer], ovn[layer], table,
                               torch.tensor([L + 1 for L in lens], dtype=torch.int32),
                               oq.Pi, oq.centroids, 4, ov.Pi, ov.centroids, 6, D)
            assert_attention_close(out, orc.tiled_attention(q, okv, D ** -0.5))
        lens = [L + 1 for L in lens]
        sess.check()
    assert sess.lengths == lens and sess.seq.tolist() == lens
    for layer in range(layers):
        assert torch.equal(pool.k_pages[layer].cpu(), okp[layer])
        assert torch.equal(pool.v_pages[layer].cpu(), ovp[layer])
        assert torch.equal(pool.k_norms[layer].cpu(), okn[layer])
        assert torch.equal(pool.v_norms[layer].cpu(), ovn[layer])
    assert pool.stats()["owned"] == 3 + 1 + 2          # 34, 4, 19 tokens on 16-token pages


def test_decode_session_refuses_to_outgrow_its_table():
    pool = PagePool(num_layers=1, num_pages=4, num_kv_heads=1, page_size=16, nb_k=64, nb_v=64, device=DEV)
    kq = _get_quantizer(4, 128, DEV, 42)
    pool.ensure("a", 16)
    sess = DecodeSession(pool, ["a"], [16], k_quant=kq, v_quant=kq, head_dim=128, q_heads=4,
                         dtype=torch.float16, max_tokens=17)
    for _ in range(16):
        sess.begin_step()                               # 17 .. 32 tokens: two pages
    with pytest.raises(StalePage):
        sess.begin_step()                               # a 33rd token needs a third page
