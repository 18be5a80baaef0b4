"""Model integration on a tiny seeded Qwen2 (random weights, fp32, head_dim 128)
through Transformers' attention interface, the harness of the reference's
turboquant_kv/test_packed_model.py:27-109 pointed at this package.

Two runs of the same model over the same prompts feed identical tokens:
* the product: `PagedPackedCache` on a GPU pool, attention = `winnow_packed`
  (chunked prefill on `wtq_prefill`, batched decode on `wtq_decode`, appends on
  `wtq_append`);
* the check: the same cache class on a second pool, attention computed by the
  CPU oracle (`orc.tiled_attention`) from the pool's bytes.
Both store their K/V through the same append kernel.  With one layer the two
pools hold identical bytes, so the logits differ only by the attention kernels'
arithmetic (bound 2e-3 relative L2).  With two layers the second layer's K/V
are quantized from hidden states that already differ by that much, a few codes
land on the other side of a bucket boundary, and the logits move by up to a
percent (measured 8e-3): that run checks the multi-layer bookkeeping against a
bound of 3e-2, which a wrong mask, head map or page (errors of order one) still
fails by a wide margin.
"""
import pytest
import torch

from oracle import tq_oracle as orc
from winnow_b200 import packed_backend as pb

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0) if torch.cuda.is_available() else None
BW = 4
ORACLE_ATTN = "winnow_oracle_check"


def _oracle_attention(module, query, key, value, attention_mask, dropout=0.0, scaling=None, **kwargs):
    """Attention-interface function: the CPU oracle on the handle's bytes."""
    kv = key
    okv = orc.OracleKV(kv.k_pages.cpu(), kv.k_norms.cpu(), kv.v_pages.cpu(), kv.v_norms.cpu(),
                       kv.page_table.cpu(), kv.seq_lens.cpu(), kv.k_quant.Pi.cpu(),
                       kv.k_quant.centroids.cpu(), kv.k_quant.bit_width, kv.v_quant.Pi.cpu(),
                       kv.v_quant.centroids.cpu(), kv.v_quant.bit_width, kv.head_dim)
    scaling = scaling if scaling is not None else query.shape[-1] ** -0.5
    out = orc.tiled_attention(query.float().cpu(), okv, scaling)          # (B, Hq, Q, D)
    return out.to(query.device, query.dtype).transpose(1, 2).contiguous(), None


@pytest.fixture(scope="module", params=[(1, 2e-3), (2, 3e-2)], ids=["one_layer", "two_layers"])
def model(request):
    from transformers import AttentionInterface, Qwen2Config, Qwen2ForCausalLM
    torch.manual_seed(0)
    layers, bound = request.param
    cfg = Qwen2Config(vocab_size=96, hidden_size=512, intermediate_size=256, num_hidden_layers=layers,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=512,
                      initializer_range=0.05, architectures=["Qwen2ForCausalLM"],
                      attn_implementation="sdpa")
    m = Qwen2ForCausalLM(cfg).eval().to(DEV)
    pb.register()
    AttentionInterface.register(ORACLE_ATTN, _oracle_attention)
    m.logit_bound = bound
    return m


def _prompts(n, seed, lo, hi):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, 96, (int(torch.randint(lo, hi, (1,), generator=g)),), generator=g).tolist()
            for _ in range(n)]


class _Run:
    """One side of the comparison: a pool, its quantizers and the lengths stored."""

    def __init__(self, model, attn: str, owners, pages=64, page_size=16):
        self.model, self.attn, self.owners = model, attn, list(owners)
        self.pool = pb.make_pool(model.config, bit_width=BW, num_pages=pages, page_size=page_size,
                                 device=DEV)
        self.kq, self.vq = pb.quantizers_for(model.config, BW, DEV)
        self.stored = {o: 0 for o in self.owners}

    @torch.no_grad()
    def forward(self, owners, ids, pos):
        self.model.config._attn_implementation = self.attn
        cache = pb.PagedPackedCache(self.pool, owners, [self.stored[o] for o in owners],
                                    k_quant=self.kq, v_quant=self.vq,
                                    head_dim=pb.head_dim_of(self.model.config))
        out = self.model(input_ids=ids, position_ids=pos, past_key_values=cache, use_cache=True,
                         logits_to_keep=1)
        cache.check()
        for o, L in zip(owners, cache.lengths):
            self.stored[o] = L
        return out.logits[:, -1].float()


def _generate(run, prompts, new_tokens, chunk, forced=None):
    """Chunked prefill of each prompt alone, then batched greedy decode; with
    `forced` the decode feeds those tokens instead of its own argmax.  Returns
    (tokens[request][step], logits[step] as (requests, vocab))."""
    owners = run.owners
    first = []
    for o, prompt in zip(owners, prompts):
        run.pool.ensure(o, len(prompt) + new_tokens)
        lo = 0
        while lo < len(prompt):
            hi = min(lo + chunk, len(prompt))
            ids = torch.tensor([prompt[lo:hi]], device=DEV)
            pos = torch.arange(lo, hi, device=DEV)[None]
            lg = run.forward([o], ids, pos)
            lo = hi
        first.append(lg[0])
    logits = [torch.stack(first)]
    toks = [[int(l.argmax())] for l in first]
    for step in range(1, new_tokens):
        feed = [forced[r][step - 1] if forced is not None else toks[r][-1] for r in range(len(owners))]
        ids = torch.tensor([[t] for t in feed], device=DEV)
        pos = torch.tensor([[run.stored[o]] for o in owners], device=DEV)
        lg = run.forward(owners, ids, pos)
        logits.append(lg)
        for r in range(len(owners)):
            toks[r].append(int(lg[r].argmax()))
    return toks, logits


def test_chunked_prefill_and_batched_decode_match_the_oracle_model(model):
    prompts = _prompts(3, seed=4, lo=20, hi=70)
    owners = ["a", "b", "c"]
    check = _Run(model, ORACLE_ATTN, owners)
    ref_toks, ref_logits = _generate(check, prompts, new_tokens=6, chunk=11)
    pb.BACKEND_COUNTS.clear()
    product = _Run(model, pb.ATTN_NAME, owners)
    toks, logits = _generate(product, prompts, new_tokens=6, chunk=11, forced=ref_toks)
    assert pb.BACKEND_COUNTS["prefill_cuda_packed"] > 0 and pb.BACKEND_COUNTS["cuda_packed"] > 0
    assert pb.BACKEND_COUNTS["prefill_reconstruct_sdpa"] == 0
    # the first layer's K/V do not depend on any attention output: same bytes in both pools
    for o in owners:
        mine = [r.page for r in product.pool.held(o)]
        theirs = [r.page for r in check.pool.held(o)]
        assert torch.equal(product.pool.k_pages[0, mine], check.pool.k_pages[0, theirs])
        assert torch.equal(product.pool.v_pages[0, mine], check.pool.v_pages[0, theirs])
        assert torch.equal(product.pool.v_norms[0, mine], check.pool.v_norms[0, theirs])
    # (a wrong mask, head map or page would move the logits by O(1))
    for got, ref in zip(logits, ref_logits):
        err = (got - ref).norm() / ref.norm()
        assert float(err) < model.logit_bound, f"logits differ by relative L2 {float(err):.2e}"
    # greedy tokens agree wherever the reference's top-2 margin exceeds the logit error
    for r in range(len(owners)):
        for step, ref in enumerate(ref_logits):
            top2 = ref[r].topk(2).values
            if float(top2[0] - top2[1]) > 4 * model.logit_bound * float(ref[r].norm()):
                assert toks[r][step] == ref_toks[r][step]
    for o in owners:
        product.pool.release(o)
    assert product.pool.stats()["owned"] == 0
