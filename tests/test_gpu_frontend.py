"""GPU parity of the projection front-end (the step in front of the indexer and the sparse attention) through the C ABI,
against fixtures made by the reference's own modules and against the oracle."""
import numpy as np
import pytest
import torch

from oracle import gw_oracle as orc
from tests import golden
from tests.gpu_util import dev

pytestmark = pytest.mark.gpu

NAMES = ["q", "k", "v", "q_idx", "k_idx", "w"]


@pytest.fixture(scope="module")
def fe_golden():
    return golden.load("reference_frontend.npz")


def T(a, dtype=None):
    t = torch.from_numpy(np.asarray(a))
    return t if dtype is None else t.to(dtype)


def params_of(c, device, table_dtype):
    from geoweave_b200.front_end import FrontEndParams

    ln = lambda w, b, eps: (T(c[w]).to(device), T(c[b]).to(device), float(c[eps]))
    return FrontEndParams(T(c["weight"]).to(device), T(c["bias"]).to(device), int(c["heads"]), 4,
                          ln("q_norm_w", "q_norm_b", "eps"), ln("k_norm_w", "k_norm_b", "eps"),
                          ln("ik_norm_w", "ik_norm_b", "ik_norm_eps"), T(c["cos"]).to(device), T(c["sin"]).to(device))


def tolerance(ref, dtype):
    # fp32: rounding order only.  16-bit: the reference rounds after every operation, this kernel once; two units in
    # the last place of the result's magnitude cover that
    if dtype == torch.float32:
        return 2e-5 + 2e-6 * ref.abs()
    return 2e-2 + 2.0 ** -7 * ref.abs()


@pytest.mark.parametrize("name,dtype", [("fe_f32", torch.float32), ("fe_bf16", torch.bfloat16), ("fe_pi3_bf16", torch.bfloat16)])
def test_epilogue_on_the_reference_linear_output(fe_golden, name, dtype):
    import geoweave_b200
    from geoweave_b200.front_end import project_epilogue

    c = fe_golden[name]
    prm = params_of(c, dev(), dtype)
    outs = project_epilogue(T(c["fused"], dtype).to(dev()), T(c["pos"]).to(dev()), prm)
    geoweave_b200.check_status()
    for nm, o in zip(NAMES, outs):
        ref = T(c[nm])
        assert o.dtype == dtype and tuple(o.shape) == tuple(ref.shape) and o.is_contiguous(), nm
        err = (o.float().cpu() - ref).abs()
        assert bool((err <= tolerance(ref, dtype)).all()), (name, nm, float(err.max()))
    assert torch.equal(outs[2].float().cpu(), T(c["v"])) and torch.equal(outs[5].float().cpu(), T(c["w"]))  # copies are exact


@pytest.mark.parametrize("name,dtype", [("fe_f32", torch.float32), ("fe_bf16", torch.bfloat16)])
def test_linear_plus_epilogue_from_the_layer_input(fe_golden, name, dtype):
    from geoweave_b200.front_end import project_qkv_and_indexer

    c = fe_golden[name]
    prm = params_of(c, dev(), dtype)
    prm.weight, prm.bias = prm.weight.to(dtype), prm.bias.to(dtype)
    outs = project_qkv_and_indexer(T(c["x"], dtype).to(dev()), T(c["pos"]).to(dev()), prm)
    for nm, o in zip(NAMES, outs):
        ref = T(c[nm])
        err = (o.float().cpu() - ref).abs()
        # the GEMM runs on another device with another summation order: one more unit in the last place
        assert bool((err <= 2 * tolerance(ref, dtype) + (1e-4 if dtype == torch.float32 else 0)).all()), (name, nm, float(err.max()))


@pytest.mark.parametrize("name", ["fe_bf16", "fe_pi3_bf16"])
def test_fused_projection_on_the_reference_fixtures(fe_golden, name):
    """x -> the six operator inputs in ONE kernel (tensor-core GEMM with the LayerNorm / rotary / layout epilogue) against
    what the reference's own modules produced from the same x and weights."""
    import geoweave_b200
    from geoweave_b200.front_end import project_fused

    c = fe_golden[name]
    dtype = torch.bfloat16
    prm = params_of(c, dev(), dtype)
    outs = project_fused(T(c["x"], dtype).to(dev()), T(c["pos"]).to(dev()), prm)
    geoweave_b200.check_status()
    for nm, o in zip(NAMES, outs):
        ref = T(c[nm])
        assert o.dtype == dtype and tuple(o.shape) == tuple(ref.shape) and o.is_contiguous(), nm
        err = (o.float().cpu() - ref).abs()
        # the reference rounds the product to bf16 before LayerNorm and after every later step, this kernel once at the end
        assert bool((err <= 2 * tolerance(ref, dtype)).all()), (name, nm, float(err.max()))


@pytest.mark.parametrize("dtype,heads,idx_heads,tokens,dim,bias,norms,rope", [
    (torch.bfloat16, 16, 4, 4164, 1024, True, True, True),    # the models' shape: 4 views
    (torch.bfloat16, 16, 4, 1000, 1024, False, False, True),  # ragged last row tile, no bias, no LayerNorm
    (torch.float16, 8, 3, 777, 256, True, True, False),       # fp16, odd number of indexer heads, no rotary embedding
    (torch.bfloat16, 3, 1, 130, 64, True, True, True),        # head slots of different kinds inside one column tile
])
def test_fused_projection_against_the_oracle(dtype, heads, idx_heads, tokens, dim, bias, norms, rope):
    """The fused kernel against the oracle's front end applied to the exact (fp32) product of the same 16-bit x and W."""
    import geoweave_b200
    from geoweave_b200.front_end import FrontEndParams, project_fused, rope_tables

    g = torch.Generator().manual_seed(tokens + heads)
    width = 3 * heads * 64 + 2 * idx_heads * 64 + idx_heads
    x = torch.randn(1, tokens, dim, generator=g).to(dtype)
    wt = (torch.randn(width, dim, generator=g) * dim ** -0.5).to(dtype)
    bs = (torch.randn(width, generator=g) * 0.2).to(dtype) if bias else None
    pos = torch.randint(0, 38, (1, tokens, 2), generator=g)
    cos, sin = rope_tables(38, "cpu", dtype)
    vec = lambda: (torch.randn(64, generator=g) * 0.3 + 1.0, torch.randn(64, generator=g) * 0.2, 1e-5)
    qn, kn, ikn = (vec(), vec(), vec()) if norms else (None, None, None)
    prm = FrontEndParams(wt.to(dev()), None if bs is None else bs.to(dev()), heads, idx_heads, qn, kn, ikn, cos, sin)
    outs = project_fused(x.to(dev()), pos.to(dev()) if rope else None, prm)
    geoweave_b200.check_status()
    fused = x.double()[0] @ wt.double().T
    if bs is not None:
        fused = fused + bs.double()
    fused = fused.float().unsqueeze(0)
    if rope:
        refs = orc.project_front_end(fused, pos, cos, sin, heads, 64, idx_heads, 64, qn, kn, ikn)
    else:
        refs = orc.project_front_end(fused, torch.zeros_like(pos), torch.ones(1, 32), torch.zeros(1, 32), heads, 64, idx_heads, 64,
                                     qn, kn, ikn)
    for nm, o, ref in zip(NAMES, outs, refs):
        assert o.dtype == dtype and tuple(o.shape) == tuple(ref.shape), nm
        err = (o.float().cpu() - ref).abs()
        ulp = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
        # one rounding to the 16-bit type; the fp32 accumulation order of the tensor cores is below that
        assert bool((err <= 1.01 * ulp * ref.abs() + 2e-3).all()), (nm, float(err.max()))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("heads,views", [(16, 8), (8, 3)])
def test_production_width_against_the_oracle(dtype, heads, views):
    """16 heads, VGGT token grid (5 special tokens at position 0 + 28 x 37 patches per view), some parts switched off."""
    from geoweave_b200.front_end import FrontEndParams, project_epilogue, rope_tables

    g = torch.Generator().manual_seed(heads * 100 + views)
    n_tok = 5 + 28 * 37
    N = views * n_tok
    width = 3 * heads * 64 + 2 * 4 * 64 + 4
    fused = (torch.randn(1, N, width, generator=g) * 1.5 + 0.3).to(dtype)
    ys, xs = torch.meshgrid(torch.arange(28), torch.arange(37), indexing="ij")
    grid = torch.stack([ys.reshape(-1), xs.reshape(-1)], -1) + 1
    pos = torch.cat([torch.zeros(5, 2, dtype=torch.int64), grid]).repeat(views, 1).view(1, N, 2)
    cos, sin = rope_tables(38, "cpu", dtype)
    vec = lambda: (torch.randn(64, generator=g) * 0.3 + 1.0, torch.randn(64, generator=g) * 0.2, 1e-5)
    prm = FrontEndParams(torch.empty(0), None, heads, 4, vec(), None if heads == 8 else vec(), vec(), cos, sin)
    outs = project_epilogue(fused.to(dev()), pos.to(dev()), prm)
    refs = orc.project_front_end(fused, pos, cos, sin, heads, 64, 4, 64, prm.q_norm, prm.k_norm, prm.idx_k_norm)
    for nm, o, ref in zip(NAMES, outs, refs):
        err = (o.float().cpu() - ref).abs()
        tol = 2e-5 + 2e-6 * ref.abs() if dtype == torch.float32 else 2.0 ** -7 * ref.abs() + 1e-3  # one unit in the last place
        assert bool((err <= tol).all()), (nm, float(err.max()))
    # without positions: no rotary embedding
    outs_np = project_epilogue(fused.to(dev()), None, prm)
    refs_np = orc.project_front_end(fused, torch.zeros_like(pos), torch.ones(1, 32), torch.zeros(1, 32), heads, 64, 4, 64,
                                    prm.q_norm, prm.k_norm, prm.idx_k_norm)
    assert (outs_np[0].float().cpu() - refs_np[0]).abs().max().item() <= (1e-4 if dtype == torch.float32 else 6e-2)


def test_front_end_feeds_the_operators_and_refuses_bad_input():
    """The six outputs go straight into the indexer and the attention; wrong widths and positions outside the
    tables are reported."""
    import geoweave_b200
    from geoweave_b200.custom_flash_attn import sparse_index_flash_attn_inference_func
    from geoweave_b200.custom_indexer import sparse_topk_indexer_inference_func
    from geoweave_b200.front_end import FrontEndParams, project_epilogue, rope_tables

    g = torch.Generator().manual_seed(9)
    N, heads = 4164, 16
    width = 3 * heads * 64 + 2 * 4 * 64 + 4
    fused = torch.randn(1, N, width, generator=g).bfloat16()
    pos = torch.randint(0, 30, (1, N, 2), generator=g)
    cos, sin = rope_tables(30, "cpu", torch.bfloat16)
    prm = FrontEndParams(torch.empty(0), None, heads, 4, None, None, None, cos, sin)
    q, k, v, qi, ki, w = project_epilogue(fused.to(dev()), pos.to(dev()), prm)
    idx, _ = sparse_topk_indexer_inference_func(qi, ki, w, None, 256, 0.125, return_scores=False)
    out, _ = sparse_index_flash_attn_inference_func(q, k, v, idx, None, False, 0.125)
    geoweave_b200.check_status()
    refs = orc.project_front_end(fused, pos, cos, sin, heads, 64, 4, 64)
    rows = torch.arange(0, N, 97)
    scores = orc.indexer_scores(refs[3].bfloat16()[:, rows], refs[4].bfloat16(), refs[5].bfloat16(), 0.125)
    res = orc.audit_topk(idx[:, rows.to(dev())], scores, 256, refs[3].bfloat16()[:, rows], refs[4].bfloat16(), refs[5].bfloat16(), 0.125)
    assert res["out_of_range"] == 0 and res["duplicates"] == 0 and res["unexplained"] == 0, res
    assert out.shape == (1, N, heads, 64) and bool(torch.isfinite(out.float()).all())
    with pytest.raises(ValueError):
        project_epilogue(fused[..., :-2].to(dev()), pos.to(dev()), prm)
    project_epilogue(fused.to(dev()), (pos + 25).to(dev()), prm)   # positions up to 54 against tables of 30 rows
    with pytest.raises(geoweave_b200.GeoWeaveError):
        geoweave_b200.check_status()


def test_whole_layer_eager_graph_and_reused_indices():
    """fused projection -> front-end -> indexer -> attention as one call; the CUDA-graph replay gives what the eager
    chain gives, and a layer that reuses another layer's indices skips its indexer."""
    import geoweave_b200
    from geoweave_b200.front_end import FrontEndParams, rope_tables
    from geoweave_b200.layer import SparseGlobalAttentionLayer

    g = torch.Generator().manual_seed(21)
    N, heads, dim, k = 8328, 16, 256, 256
    width = 3 * heads * 64 + 2 * 4 * 64 + 4
    weight = (torch.randn(width, dim, generator=g) * dim ** -0.5).bfloat16().to(dev())
    bias = (torch.randn(width, generator=g) * 0.1).bfloat16().to(dev())
    cos, sin = rope_tables(40, dev(), torch.bfloat16)
    vec = lambda: ((torch.rand(64, generator=g) + 0.5).to(dev()), (torch.randn(64, generator=g) * 0.1).to(dev()), 1e-5)
    prm = FrontEndParams(weight, bias, heads, 4, vec(), vec(), vec(), cos, sin)
    eager = SparseGlobalAttentionLayer(prm, k)
    graphed = SparseGlobalAttentionLayer(prm, k, use_cuda_graph=True)
    for trial in range(2):
        x = torch.randn(1, N, dim, generator=g).bfloat16().to(dev())
        pos = torch.randint(0, 40, (1, N, 2), generator=g).to(dev())
        out_e, idx_e = eager(x, pos)
        out_g, idx_g = graphed(x, pos)
        geoweave_b200.check_status()
        assert out_e.shape == (1, N, heads * 64) and idx_e.shape == (1, N, k)
        assert torch.equal(torch.sort(idx_e.long(), -1).values, torch.sort(idx_g.long(), -1).values)
        assert (out_e.float() - out_g.float()).abs().max().item() <= 2e-2
        # a second layer on the same tokens that takes these indices: same attention as handing them over by hand
        out_r, idx_r = eager(x, pos, reuse_topk_indices=idx_e)
        assert idx_r.data_ptr() == idx_e.data_ptr() or torch.equal(idx_r, idx_e)
        assert (out_r.float() - out_e.float()).abs().max().item() <= 2e-2
        out_rg, _ = graphed(x, pos, reuse_topk_indices=idx_e)
        assert (out_rg.float() - out_e.float()).abs().max().item() <= 2e-2
    with pytest.raises(ValueError):
        eager(x, pos, reuse_topk_indices=idx_e[:, :10])
    # the chain against the oracle, stage by stage on the chain's own intermediate tensors: the indices the layer
    # returned are an exact top-k of the oracle's scores, and its output is the oracle's attention over them
    from geoweave_b200.front_end import project_qkv_and_indexer

    q, kk, v, qi, ki, w = [t.cpu() for t in project_qkv_and_indexer(x, pos, prm)]
    rows = torch.arange(0, N, 61)
    scores = orc.indexer_scores(qi[:, rows], ki, w, 0.125)
    res = orc.audit_topk(idx_g[:, rows.to(dev())], scores, k, qi[:, rows], ki, w, 0.125)
    assert res["out_of_range"] == 0 and res["duplicates"] == 0 and res["unexplained"] == 0, res
    ref_out, _, _ = orc.sparse_attention(q[:, rows], kk, v, idx_g[:, rows.to(dev())].cpu(), 0.125)
    got = out_g.view(1, N, heads, 64)[:, rows.to(dev())].float().cpu()
    assert (got - ref_out).abs().max().item() <= 2e-2


def test_a_captured_layer_survives_later_calls_that_replace_the_cached_workspace():
    """A graph records raw pointers.  The layer's graph owns its indexer workspace, so a later, larger eager call
    (which replaces the per-stream cached workspace) and clear_runtime_cache() cannot pull it from under a replay."""
    import geoweave_b200
    from geoweave_b200.front_end import FrontEndParams, rope_tables
    from geoweave_b200.layer import SparseGlobalAttentionLayer

    g = torch.Generator().manual_seed(33)
    heads, dim, k = 16, 128, 128
    width = 3 * heads * 64 + 2 * 4 * 64 + 4
    weight = (torch.randn(width, dim, generator=g) * dim ** -0.5).bfloat16().to(dev())
    cos, sin = rope_tables(40, dev(), torch.bfloat16)
    prm = FrontEndParams(weight, None, heads, 4, None, None, None, cos, sin)
    eager = SparseGlobalAttentionLayer(prm, k)
    graphed = SparseGlobalAttentionLayer(prm, k, use_cuda_graph=True)
    mk = lambda n: (torch.randn(1, n, dim, generator=g).bfloat16().to(dev()), torch.randint(0, 40, (1, n, 2), generator=g).to(dev()))
    xa, pa = mk(5000)                      # shape A: large enough for the sampled fast path (lists in the workspace)
    out_a, idx_a = [t.clone() for t in graphed(xa, pa)]
    xb, pb = mk(9000)                      # a larger shape B through the shared cache, then the cache is dropped
    eager(xb, pb)
    geoweave_b200.clear_runtime_cache()
    junk = [torch.full((1 << 24,), 0x7f, dtype=torch.uint8, device=dev()) for _ in range(8)]  # reuse freed blocks
    xa2, pa2 = mk(5000)
    out_r, idx_r = graphed(xa2, pa2)       # replay of A with new inputs
    out_e, idx_e = eager(xa2, pa2)
    geoweave_b200.check_status()
    del junk
    assert torch.equal(torch.sort(idx_r.long(), -1).values, torch.sort(idx_e.long(), -1).values)
    assert (out_r.float() - out_e.float()).abs().max().item() <= 2e-2
    assert not torch.equal(out_r, out_a)
