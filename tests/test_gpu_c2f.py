"""GPU parity of the coarse-to-fine selection: pooled sources and expansion against the reference's own outputs
(``tests/golden/reference_c2f.npz``) and, on larger seeded inputs, against the oracle; the whole selection against the
oracle's pipeline; the layer with pooled sources."""
import numpy as np
import pytest
import torch

import geoweave_b200
from geoweave_b200.coarse_to_fine import expand_sources, pool_sources, select_topk_coarse_to_fine, source_layout
from oracle import gw_oracle as orc
from tests import golden
from tests.golden.make_golden_c2f import CASES
from tests.gpu_util import dev

pytestmark = pytest.mark.gpu
GOLD = golden.load("reference_c2f.npz")


@pytest.mark.parametrize("name", [n for n in sorted(CASES) if CASES[n][7]])
def test_pooled_sources_match_the_reference(name):
    tpv, views, special, gh, gw, _, _, _ = CASES[name]
    lay = source_layout(tpv, views, special, gh, gw, dev())
    g = GOLD[name]
    k, w = torch.from_numpy(g["k"]).to(dev()), torch.from_numpy(g["w"]).to(dev())
    sk, sw = pool_sources(k, w, lay)                           # fp32 in, fp32 out
    assert np.allclose(sk.cpu().numpy(), g["src_k"], rtol=0, atol=1e-6) and np.allclose(sw.cpu().numpy(), g["src_w"], rtol=0, atol=1e-6)
    for dt in (torch.bfloat16, torch.float16):                 # 16-bit in (exactly representable), mean rounded once
        sk, sw = pool_sources(k.to(dt), w.to(dt), lay)
        ref_k, ref_w = torch.from_numpy(g["src_k"]).to(dt), torch.from_numpy(g["src_w"]).to(dt)
        if dt == torch.bfloat16:
            assert torch.equal(sk.cpu(), ref_k) and torch.equal(sw.cpu(), ref_w)
        else:  # the fixture's inputs are bf16 values, not all exact in fp16
            kk, ww = orc.pool_sources(k.to(dt).cpu(), w.to(dt).cpu(), orc.source_layout(tpv, views, special, gh, gw))
            assert torch.equal(sk.cpu(), kk.to(dt)) and torch.equal(sw.cpu(), ww.to(dt))


@pytest.mark.parametrize("name", sorted(CASES))
def test_expansion_in_the_given_order_matches_the_reference(name):
    tpv, views, special, gh, gw, topk, _, _ = CASES[name]
    lay = source_layout(tpv, views, special, gh, gw, dev())
    g = GOLD[name]
    fine = expand_sources(torch.from_numpy(g["lists"]).to(dev()), None, lay, topk)
    assert fine.dtype == torch.int32 and np.array_equal(fine.cpu().numpy(), g["fine"])


@pytest.mark.parametrize("tpv,views,special,gh,gw,topk,m,dt", [
    (5 + 28 * 37, 3, 5, 28, 37, 1024, 300, torch.bfloat16),
    (5 + 21 * 37, 2, 5, 21, 37, 512, 149, torch.float32),
    (2 + 5 * 7, 2, 2, 5, 7, 60, 11, torch.float16),            # short lists: padded
    (1 + 6 * 6, 4, 1, 6, 6, 100, 40, torch.bfloat16),          # more tokens than wanted: cut inside a slot round
])
def test_expansion_by_descending_score(tpv, views, special, gh, gw, topk, m, dt):
    lay = source_layout(tpv, views, special, gh, gw, dev())
    olay = orc.source_layout(tpv, views, special, gh, gw)
    g = torch.Generator().manual_seed(m)
    T = 70
    lists = torch.stack([torch.stack([torch.randperm(lay.source_len, generator=g)[:m] for _ in range(T)]) for _ in range(2)]).to(torch.int32)
    scores = (torch.randn(2, T, m, generator=g) * 3).round().div(2).to(dt)   # many equal scores
    fine = expand_sources(lists.to(dev()), scores.to(dev()), lay, topk)
    # oracle: stable sort by (score descending, source ascending), then the reference's expansion of the ordered list
    by_src = torch.argsort(lists.long(), dim=-1, stable=True)
    l1, s1 = torch.gather(lists.long(), -1, by_src), torch.gather(scores.float(), -1, by_src)
    by_score = torch.argsort(s1, dim=-1, descending=True, stable=True)
    ordered = torch.gather(l1, -1, by_score)
    want = orc.expand_sources(ordered, olay, topk, tpv * views)
    assert torch.equal(fine.cpu().long(), want)


def test_whole_selection_against_the_oracle_pipeline():
    tpv, views, special, gh, gw, topk = 5 + 28 * 37, 2, 5, 28, 37, 256
    lay = source_layout(tpv, views, special, gh, gw, dev())
    olay = orc.source_layout(tpv, views, special, gh, gw)
    N = tpv * views
    g = torch.Generator().manual_seed(7)
    q = torch.randn(1, N, 4, 64, generator=g).bfloat16()
    k = torch.randn(1, N, 4, 64, generator=g).bfloat16()
    w = torch.rand(1, N, 4, generator=g).bfloat16()
    idx = select_topk_coarse_to_fine(q.to(dev()), k.to(dev()), w.to(dev()), lay, topk, 0.125)
    geoweave_b200.check_status()
    assert tuple(idx.shape) == (1, N, topk) and int(idx.min()) >= 0 and int(idx.max()) < N
    # stage by stage with the oracle: pooled sources (rounded to bf16 as the kernel stores them), exact top-m of the
    # oracle's scores, expansion by descending score
    sk, sw = orc.pool_sources(k, w, olay)
    sk, sw = sk.bfloat16(), sw.bfloat16()
    m = lay.kept_sources(topk)
    assert m == orc.coarse_topk(olay, topk)
    rows = torch.arange(0, N, 9)
    from geoweave_b200.custom_indexer.sparse_topk_indexer import fused_score_topk
    kept, sc = fused_score_topk(q.to(dev())[:, rows.to(dev())], sk.to(dev()), sw.to(dev()), m, 0.125, return_scores=True)
    scores = orc.indexer_scores(q[:, rows], sk, sw, 0.125)
    res = orc.audit_topk(kept.cpu(), scores, m, q[:, rows], sk, sw, 0.125)
    assert res["out_of_range"] == 0 and res["duplicates"] == 0 and res["unexplained"] == 0, res
    by_src = torch.argsort(kept.cpu().long(), dim=-1, stable=True)
    l1, s1 = torch.gather(kept.cpu().long(), -1, by_src), torch.gather(sc.cpu().float(), -1, by_src)
    ordered = torch.gather(l1, -1, torch.argsort(s1, dim=-1, descending=True, stable=True))
    want = orc.expand_sources(ordered, olay, topk, N)
    assert torch.equal(idx.cpu()[:, rows].long(), want)


def test_layer_with_pooled_sources_eager_and_graph():
    """The whole layer with a source layout: the indices are what the coarse-to-fine selection gives on the layer's own
    projections, the CUDA-graph replay gives what the eager chain gives, and the output is the attention over them."""
    from geoweave_b200.front_end import FrontEndParams, project_qkv_and_indexer, rope_tables
    from geoweave_b200.layer import SparseGlobalAttentionLayer

    g = torch.Generator().manual_seed(17)
    tpv, views, special, gh, gw = 5 + 28 * 37, 4, 5, 28, 37
    N, heads, dim, k = tpv * views, 16, 256, 512
    lay = source_layout(tpv, views, special, gh, gw, dev())
    width = 3 * heads * 64 + 2 * 4 * 64 + 4
    weight = (torch.randn(width, dim, generator=g) * dim ** -0.5).bfloat16().to(dev())
    cos, sin = rope_tables(40, dev(), torch.bfloat16)
    vec = lambda: ((torch.rand(64, generator=g) + 0.5).to(dev()), (torch.randn(64, generator=g) * 0.1).to(dev()), 1e-5)
    prm = FrontEndParams(weight, None, heads, 4, vec(), vec(), vec(), cos, sin)
    eager = SparseGlobalAttentionLayer(prm, k, source_layout=lay)
    graphed = SparseGlobalAttentionLayer(prm, k, use_cuda_graph=True, source_layout=lay)
    x = torch.randn(1, N, dim, generator=g).bfloat16().to(dev())
    ys, xs = torch.meshgrid(torch.arange(gh), torch.arange(gw), indexing="ij")
    grid = torch.stack([ys.reshape(-1), xs.reshape(-1)], -1) + 1
    pos = torch.cat([torch.zeros(special, 2, dtype=torch.long), grid]).repeat(views, 1).view(1, N, 2).to(dev())
    for trial in range(2):
        out_e, idx_e = eager(x, pos)
        out_g, idx_g = graphed(x, pos)
        geoweave_b200.check_status()
        assert idx_e.shape == (1, N, k) and torch.equal(idx_e, idx_g)   # the expansion fixes the order too
        assert (out_e.float() - out_g.float()).abs().max().item() <= 2e-2
        x = x.roll(1, 1)
    q, kk, v, qi, ki, w = project_qkv_and_indexer(x.roll(-1, 1), pos, prm)
    want = select_topk_coarse_to_fine(qi, ki, w, lay, k, 0.125)
    assert torch.equal(want, idx_g)
    rows = torch.arange(0, N, 97)
    ref_out, _, _ = orc.sparse_attention(q.cpu()[:, rows], kk.cpu(), v.cpu(), idx_g[:, rows.to(dev())].cpu(), 0.125)
    got = out_g.view(1, N, heads, 64)[:, rows.to(dev())].float().cpu()
    assert (got - ref_out).abs().max().item() <= 2e-2


def test_pooled_queries_take_their_cells_list():
    """qk_sym_x2_broadcast: queries pooled like the keys (checked against the reference's pooled queries), one list per
    source, every token takes its source's list."""
    name = "vggt1"
    tpv, views, special, gh, gw, _, _, _ = CASES[name]
    lay = source_layout(tpv, views, special, gh, gw, dev())
    olay = orc.source_layout(tpv, views, special, gh, gw)
    g = GOLD[name]
    k = torch.from_numpy(g["k"]).to(dev())
    cq, none = pool_sources(k, None, lay)
    assert none is None and np.allclose(cq.cpu().numpy(), g["coarse_q"], rtol=0, atol=1e-6)
    assert np.array_equal(lay.token_source.cpu().numpy(), g["fine_to_row"])
    N, topk = tpv * views, 128
    gen = torch.Generator().manual_seed(3)
    q = torch.randn(1, N, 4, 64, generator=gen).bfloat16().to(dev())
    kk = torch.randn(1, N, 4, 64, generator=gen).bfloat16().to(dev())
    w = torch.rand(1, N, 4, generator=gen).bfloat16().to(dev())
    idx = select_topk_coarse_to_fine(q, kk, w, lay, topk, 0.125, pool_queries=True)
    geoweave_b200.check_status()
    assert tuple(idx.shape) == (1, N, topk) and idx.dtype == torch.int32
    # one list per source, from the pooled queries scored against the pooled keys
    sq, _ = pool_sources(q, None, lay)
    sk, sw = pool_sources(kk, w, lay)
    lists = select_topk_coarse_to_fine(sq, kk, w, lay, topk, 0.125)          # pooled queries as an ordinary query block
    assert torch.equal(idx, lists.index_select(1, lay.token_source))
    src = orc.token_source(olay)
    assert torch.equal(idx.cpu()[0, 7], lists.cpu()[0, src[7]])
    # and those lists against the oracle's scores of the oracle's pooled queries
    oq, _ = orc.pool_sources(q.cpu(), w.cpu(), olay)
    assert torch.equal(sq.cpu(), oq.bfloat16())
    from geoweave_b200.custom_indexer.sparse_topk_indexer import fused_score_topk
    m = lay.kept_sources(topk)
    kept, _ = fused_score_topk(sq, sk, sw, m, 0.125, return_scores=True)
    res = orc.audit_topk(kept.cpu(), orc.indexer_scores(sq.cpu(), sk.cpu(), sw.cpu(), 0.125), m, sq.cpu(), sk.cpu(), sw.cpu(), 0.125)
    assert res["out_of_range"] == 0 and res["duplicates"] == 0 and res["unexplained"] == 0, res
