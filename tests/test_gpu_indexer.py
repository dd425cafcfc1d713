"""GPU parity: tcgen05 indexer scores and the fused score + exact top-k, through the C ABI."""
import pytest
import torch

import geoweave_b200
from oracle import gw_oracle as orc
from tests.gpu_util import dev, make_indexer_inputs, sorted_idx, t

pytestmark = pytest.mark.gpu

EXACT_CASES = ["idx_int", "idx_int_ties"]          # every partial sum exact in fp32: bit-exact whatever the order
FLOAT_CASES = ["idx_bf16", "idx_bf16_ties", "idx_negw", "idx_kgeS"]


def _inputs(c, dtype=torch.bfloat16):
    return t(c["q_idx"], dtype), t(c["k_idx"], dtype), t(c["w"], dtype)


@pytest.mark.parametrize("name", EXACT_CASES + FLOAT_CASES)
def test_dense_scores_match_reference(golden, name):
    from geoweave_b200.custom_indexer.sparse_topk_indexer import indexer_scores

    c = golden[name]
    q, k, w = _inputs(c)
    sc = indexer_scores(q, k, w, float(c["scale"]))
    geoweave_b200.check_status()
    ref = torch.from_numpy(c["scores"])
    if name in EXACT_CASES:
        assert torch.equal(sc.cpu(), ref)
    else:
        bound = 64 * 2.0**-24 * float(ref.abs().max()) * 8
        assert (sc.cpu() - ref).abs().max().item() <= bound


@pytest.mark.parametrize("step", [3, 7])
def test_dense_scores_with_key_step(golden, step):
    from geoweave_b200.custom_indexer.sparse_topk_indexer import indexer_scores

    c = golden["idx_int_ties"]
    q, k, w = _inputs(c)
    sc = indexer_scores(q, k, w, float(c["scale"]), key_step=step)
    assert torch.equal(sc.cpu(), torch.from_numpy(c["scores"])[..., ::step])


@pytest.mark.parametrize("name", EXACT_CASES)
def test_fused_topk_bit_exact_on_exact_inputs(golden, name):
    from geoweave_b200.custom_indexer import sparse_topk_indexer_func

    c = golden[name]
    q, k, w = _inputs(c)
    idx, sc = sparse_topk_indexer_func(q, k, w, q.new_empty(0), int(c["k"]), float(c["scale"]), 256)
    geoweave_b200.check_status()
    assert idx.dtype == torch.int32 and sc.dtype == q.dtype
    assert torch.equal(sorted_idx(idx), torch.from_numpy(c["tie_idx"]).long())
    ref_sc = torch.from_numpy(c["scores"]).gather(-1, idx.long().cpu())
    assert torch.equal(sc.float().cpu(), ref_sc.bfloat16().float())


@pytest.mark.parametrize("name", FLOAT_CASES)
def test_fused_topk_on_float_inputs_audited(golden, name):
    from geoweave_b200.custom_indexer import sparse_topk_indexer_inference_func

    c = golden[name]
    q, k, w = _inputs(c)
    kk = min(int(c["k"]), k.shape[1])
    idx, none = sparse_topk_indexer_inference_func(q, k, w, None, int(c["k"]), float(c["scale"]), 256, 0, return_scores=False)
    geoweave_b200.check_status()
    assert none is None and idx.shape[-1] == kk
    res = orc.audit_topk(idx, c["scores"], kk, c["q_idx"], c["k_idx"], c["w"], float(c["scale"]))
    assert res["out_of_range"] == 0 and res["duplicates"] == 0 and res["unexplained"] == 0, res


def test_same_scores_selection_is_bit_identical(golden):
    """Scores made by the tensor-core kernel, selection by the fused epilogue vs the oracle on THOSE scores."""
    from geoweave_b200.custom_indexer import sparse_topk_indexer_func
    from geoweave_b200.custom_indexer.sparse_topk_indexer import indexer_scores

    for seed, (T, S, k, ties) in enumerate([(300, 4164, 1024, False), (200, 5000, 64, True), (129, 1041, 512, True)]):
        q, kx, w = [x.to(dev()) for x in make_indexer_inputs(T, S, seed=seed, ties=ties)]
        dense = indexer_scores(q, kx, w, 0.125)
        idx, sc = sparse_topk_indexer_func(q, kx, w, None, k, 0.125, 256)
        geoweave_b200.check_status()
        expect = orc.topk_tie_exact(dense.cpu(), k)
        assert torch.equal(sorted_idx(idx), expect.long()), (T, S, k)


@pytest.mark.parametrize("T,S,k,kind", [
    (256, 8328, 256, "randn"),      # sampled threshold path (S >= 8k)
    (256, 8328, 512, "ties"),
    (200, 16656, 1024, "integer"),
    (130, 33312, 1024, "randn"),
    (130, 33312, 2048, "ties"),
    (64, 4164, 1024, "randn"),      # streaming path (top 25 %)
    (64, 2082, 2048, "integer"),
])
def test_fused_topk_at_scale(T, S, k, kind):
    from geoweave_b200.custom_indexer import sparse_topk_indexer_func

    q, kx, w = make_indexer_inputs(T, S, seed=T + S + k, ties=(kind == "ties"), integer=(kind == "integer"))
    idx, sc = sparse_topk_indexer_func(q.to(dev()), kx.to(dev()), w.to(dev()), None, k, 0.125, 256)
    geoweave_b200.check_status()
    scores = orc.indexer_scores(q, kx, w, 0.125)
    if kind == "integer":
        assert torch.equal(sorted_idx(idx), orc.topk_tie_exact(scores, k).long())
    else:
        res = orc.audit_topk(idx, scores, k, q, kx, w, 0.125)
        assert res["out_of_range"] == 0 and res["duplicates"] == 0 and res["unexplained"] == 0, res
        assert res["rows_equal"] >= 0.95 * res["rows"], res


def test_adversarial_key_order_still_exact():
    """Keys sorted so that scores rise with the index: the sampled threshold is useless and every list keeps
    overflowing; the result must still be exact."""
    from geoweave_b200.custom_indexer import sparse_topk_indexer_func

    T, S, k = 128, 8328, 256
    g = torch.Generator().manual_seed(9)
    q = torch.randint(0, 3, (1, T, 4, 64), generator=g).float()
    kx = torch.randint(0, 3, (1, S, 4, 64), generator=g).float()
    w = (torch.arange(S).float() // 16 / 1024).view(1, S, 1).expand(1, S, 4).contiguous()
    q, kx, w = q.bfloat16(), kx.bfloat16(), w.bfloat16()
    idx, _ = sparse_topk_indexer_func(q.to(dev()), kx.to(dev()), w.to(dev()), None, k, 0.125, 256)
    geoweave_b200.check_status()
    assert torch.equal(sorted_idx(idx), orc.topk_tie_exact(orc.indexer_scores(q, kx, w, 0.125), k).long())


def test_all_equal_scores_pick_the_lowest_indices():
    from geoweave_b200.custom_indexer import sparse_topk_indexer_func

    T, S, k = 70, 5000, 300
    q = torch.zeros(1, T, 4, 64).bfloat16()
    kx = torch.ones(1, S, 4, 64).bfloat16()
    w = torch.ones(1, S, 4).bfloat16()
    idx, sc = sparse_topk_indexer_func(q.to(dev()), kx.to(dev()), w.to(dev()), None, k, 0.125, 256)
    geoweave_b200.check_status()
    assert torch.equal(sorted_idx(idx), torch.arange(k).expand(1, T, k))
    assert float(sc.abs().max()) == 0.0


def test_fp16_inputs_and_fewer_heads():
    from geoweave_b200.custom_indexer import sparse_topk_indexer_func

    for Hi in (1, 2, 3):
        q, kx, w = make_indexer_inputs(100, 700, Hi=Hi, seed=Hi, dtype=torch.float16, integer=True)
        idx, _ = sparse_topk_indexer_func(q.to(dev()), kx.to(dev()), w.to(dev()), None, 50, 0.125, 256)
        geoweave_b200.check_status()
        assert torch.equal(sorted_idx(idx), orc.topk_tie_exact(orc.indexer_scores(q, kx, w, 0.125), 50).long())


def test_unsupported_arguments_fail_loudly():
    from geoweave_b200.custom_indexer import sparse_topk_indexer_func
    from geoweave_b200.custom_indexer.score_topk_fused_cuda import score_topk_fused_select

    q, kx, w = [x.to(dev()) for x in make_indexer_inputs(10, 40, Hi=2, Di=32)]
    with pytest.raises(geoweave_b200.GeoWeaveError):
        sparse_topk_indexer_func(q, kx, w, None, 8, None, 0)  # head dim 32 has no kernel and no fallback
    q, kx, w = [x.to(dev()) for x in make_indexer_inputs(10, 40)]
    with pytest.raises(NotImplementedError):
        sparse_topk_indexer_func(q, kx, w, torch.zeros(1, 10, 40, device=dev()), 8, None, 0)
    with pytest.raises(TypeError):
        sparse_topk_indexer_func(q.double(), kx.double(), w.double(), None, 8, None, 0)
    with pytest.raises(TypeError):
        sparse_topk_indexer_func(q.float(), kx, w, None, 8, None, 0)  # mixed dtypes
    sc, pos = score_topk_fused_select(q, kx, w, softmax_scale=0.125, out_pos=torch.empty(1, 10, 16, dtype=torch.int32, device=dev()))
    assert pos.shape == (1, 10, 16) and sc.shape == (1, 10, 16)


def test_fp32_operands_small_cases_are_exact_on_integer_inputs():
    """fp32 q_idx/k_idx/w (the reference's torch backend): FFMA score kernel + exact top-k kernel.  Integer-valued
    inputs make every partial sum exact, so the selection must equal the oracle's bit for bit; ragged sizes."""
    from geoweave_b200.custom_indexer import sparse_topk_indexer_func
    from geoweave_b200.custom_indexer.sparse_topk_indexer import indexer_scores

    for T, S, k, Hi in ((1, 64, 64, 4), (77, 130, 40, 3), (300, 5000, 512, 4), (65, 4097, 1024, 1)):
        q, kx, w = make_indexer_inputs(T, S, Hi=Hi, seed=T + S, dtype=torch.float32, integer=True)
        sc = indexer_scores(q.to(dev()), kx.to(dev()), w.to(dev()), 0.125)
        ref_sc = orc.indexer_scores(q, kx, w, 0.125)
        assert torch.equal(sc.cpu(), ref_sc), (T, S)
        idx, top = sparse_topk_indexer_func(q.to(dev()), kx.to(dev()), w.to(dev()), None, k, 0.125, 256)
        geoweave_b200.check_status()
        assert idx.dtype == torch.int32 and top.dtype == torch.float32
        assert torch.equal(sorted_idx(idx), orc.topk_tie_exact(ref_sc, k).long()), (T, S)
        assert torch.equal(top.cpu(), ref_sc.gather(-1, idx.cpu().long()))
    qa, ka, wa = make_indexer_inputs(70, 900, seed=71, dtype=torch.float32, integer=True)
    qb, kb, wb = make_indexer_inputs(70, 900, seed=72, dtype=torch.float32, integer=True)
    q, kx, w = torch.cat([qa, qb]), torch.cat([ka, kb]), torch.cat([wa, wb])
    idx, _ = sparse_topk_indexer_func(q.to(dev()), kx.to(dev()), w.to(dev()), None, 100, 0.125, 256)
    assert torch.equal(sorted_idx(idx), orc.topk_tie_exact(orc.indexer_scores(q, kx, w, 0.125), 100).long())


def test_config1_in_fp32_end_to_end_at_full_size():
    """The reference's CPU-runnable configuration as written: fp32, 4 views, N = 4164, 16 x 64 attention heads,
    4 x 64 indexer heads, w ~ U(0,1), k = 1024.  Indices audited against the oracle on every row (an fp32 product
    rounds, unlike a bf16 one, so the bound allows one more rounding per term); attention within 1e-4."""
    from geoweave_b200.custom_flash_attn import sparse_index_flash_attn_inference_func
    from geoweave_b200.custom_indexer import sparse_topk_indexer_func

    N, k = 4164, 1024
    g = torch.Generator().manual_seed(1235)
    q, kk, v = [torch.randn(1, N, 16, 64, generator=g) for _ in range(3)]
    q_idx, k_idx = torch.randn(1, N, 4, 64, generator=g), torch.randn(1, N, 4, 64, generator=g)
    w = torch.rand(1, N, 4, generator=g)
    idx, _ = sparse_topk_indexer_func(q_idx.to(dev()), k_idx.to(dev()), w.to(dev()), None, k, 0.125, 256)
    out, _ = sparse_index_flash_attn_inference_func(q.to(dev()), kk.to(dev()), v.to(dev()), idx, None, False, 0.125, False)
    geoweave_b200.check_status()
    scores = orc.indexer_scores(q_idx, k_idx, w, 0.125)
    res = orc.audit_topk(idx, scores, k, q_idx, k_idx, w, 0.125, c=130.0)
    assert res["out_of_range"] == 0 and res["duplicates"] == 0 and res["unexplained"] == 0, res
    assert res["rows_equal"] >= 0.98 * N, res
    rows = torch.arange(0, N, 4)
    ref, _, _ = orc.sparse_attention(q[:, rows], kk, v, idx[:, rows.to(dev())].cpu(), 0.125)
    assert (out[:, rows.to(dev())].cpu() - ref).abs().max().item() <= 1e-4


def _finalize_counters():
    """[overflowed, short, general, lean] rows seen by the finalize kernel since the last call."""
    import ctypes

    from geoweave_b200 import _lib

    buf = (ctypes.c_ulonglong * 4)()
    assert _lib.load().gw_debug_indexer_profile(buf, 4) == 4
    return list(buf)


def test_fast_path_is_the_one_that_runs_and_needs_no_redo():
    """Large key set, generic data: every row is finished by the lean selection, none is flagged for the redo pass."""
    from geoweave_b200.custom_indexer import sparse_topk_indexer_func

    q, kx, w = make_indexer_inputs(384, 16656, seed=77)
    _finalize_counters()
    idx, _ = sparse_topk_indexer_func(q.to(dev()), kx.to(dev()), w.to(dev()), None, 512, 0.125, 256)
    geoweave_b200.check_status()
    overflowed, short, general, lean = _finalize_counters()
    assert (overflowed, short) == (0, 0) and general + lean == 384 and lean >= 380
    res = orc.audit_topk(idx, orc.indexer_scores(q, kx, w, 0.125), 512, q, kx, w, 0.125)
    assert res["unexplained"] == 0 and res["duplicates"] == 0, res


def test_fast_path_heavy_ties_use_the_general_selection():
    """Scores take few distinct values (small integers): the boundary bin of the lean selection is crowded, the
    general routine takes over, and the lower-index rule still holds exactly."""
    from geoweave_b200.custom_indexer import sparse_topk_indexer_func

    g = torch.Generator().manual_seed(5)
    T, S, k = 256, 8328, 512
    q = torch.randint(0, 2, (1, T, 4, 64), generator=g).float().bfloat16()
    kx = torch.randint(0, 2, (1, S, 4, 64), generator=g).float().bfloat16()
    w = torch.ones(1, S, 4).bfloat16()
    _finalize_counters()
    idx, _ = sparse_topk_indexer_func(q.to(dev()), kx.to(dev()), w.to(dev()), None, k, 0.125, 256)
    geoweave_b200.check_status()
    counters = _finalize_counters()
    assert torch.equal(sorted_idx(idx), orc.topk_tie_exact(orc.indexer_scores(q, kx, w, 0.125), k).long()), counters


def test_fast_path_shortfall_and_overflow_rows_are_redone_exactly():
    """Half of the keys carry a huge weight only in the second half of the key order, the sample sees them, but a
    few query rows are all-zero (every score ties at 0): whatever the filter does with such rows, the result is exact."""
    from geoweave_b200.custom_indexer import sparse_topk_indexer_func

    g = torch.Generator().manual_seed(6)
    T, S, k = 200, 9000, 256
    q = torch.randn(1, T, 4, 64, generator=g)
    q[0, ::7] = 0.0  # rows whose scores are all exactly 0
    kx = torch.randn(1, S, 4, 64, generator=g)
    w = torch.rand(1, S, 4, generator=g)
    w[0, S // 2:] *= 50.0
    q, kx, w = q.bfloat16(), kx.bfloat16(), w.bfloat16()
    idx, _ = sparse_topk_indexer_func(q.to(dev()), kx.to(dev()), w.to(dev()), None, k, 0.125, 256)
    geoweave_b200.check_status()
    scores = orc.indexer_scores(q, kx, w, 0.125)
    res = orc.audit_topk(idx, scores, k, q, kx, w, 0.125)
    assert res["out_of_range"] == 0 and res["duplicates"] == 0 and res["unexplained"] == 0, res
    zero_rows = sorted_idx(idx)[0, ::7]
    assert torch.equal(zero_rows, torch.arange(k).expand(zero_rows.shape[0], k))  # all ties: the k lowest indices


def test_long_key_set_few_queries():
    """T != S with a key set of 133248 (128 views): the chunked sample / filter / finalize path."""
    from geoweave_b200.custom_indexer import sparse_topk_indexer_func

    q, kx, w = make_indexer_inputs(130, 133248, seed=8)
    idx, _ = sparse_topk_indexer_func(q.to(dev()), kx.to(dev()), w.to(dev()), None, 1024, 0.125, 256)
    geoweave_b200.check_status()
    res = orc.audit_topk(idx, orc.indexer_scores(q, kx, w, 0.125), 1024, q, kx, w, 0.125)
    assert res["out_of_range"] == 0 and res["duplicates"] == 0 and res["unexplained"] == 0, res


@pytest.mark.parametrize("Hi,dtype", [(1, torch.bfloat16), (2, torch.float16), (3, torch.bfloat16), (4, torch.float16)])
def test_fast_path_other_head_counts_and_fp16(Hi, dtype):
    from geoweave_b200.custom_indexer import sparse_topk_indexer_func

    q, kx, w = make_indexer_inputs(150, 8328, Hi=Hi, seed=40 + Hi, dtype=dtype, integer=True)
    _finalize_counters()
    idx, sc = sparse_topk_indexer_func(q.to(dev()), kx.to(dev()), w.to(dev()), None, 256, 0.125, 256)
    geoweave_b200.check_status()
    assert sum(_finalize_counters()) == 150  # went through the fast path's finalize kernel
    scores = orc.indexer_scores(q, kx, w, 0.125)
    assert torch.equal(sorted_idx(idx), orc.topk_tie_exact(scores, 256).long())
    assert torch.equal(sc.float().cpu(), scores.gather(-1, idx.long().cpu()).to(dtype).float())


def test_batch_of_two_on_the_fast_path():
    from geoweave_b200.custom_indexer import sparse_topk_indexer_func

    qa, ka, wa = make_indexer_inputs(140, 8328, seed=51, integer=True)
    qb, kb, wb = make_indexer_inputs(140, 8328, seed=52, integer=True)
    q, kx, w = torch.cat([qa, qb]), torch.cat([ka, kb]), torch.cat([wa, wb])
    idx, _ = sparse_topk_indexer_func(q.to(dev()), kx.to(dev()), w.to(dev()), None, 300, 0.125, 256)
    geoweave_b200.check_status()
    assert torch.equal(sorted_idx(idx), orc.topk_tie_exact(orc.indexer_scores(q, kx, w, 0.125), 300).long())


@pytest.mark.parametrize("N,k,ties,n_audit", [
    (33312, 1024, False, 1024),   # 32 views, every row a query: the benchmark's shape
    (33312, 2048, True, 384),     # 10 % duplicated key rows
    (133248, 1024, False, 384),   # 128 views
    (532992, 1024, False, 160),   # 512 views: several row chunks, 8328 key tiles
    (532992, 256, False, 96),     # small k against a long key set: many sampled keys, chunks bounded by the sample buffer
])
def test_full_size_self_selection(N, k, ties, n_audit):
    """T = S at full size.  Whole output: k distinct in-range indices per row.  Sampled rows (tile edges, first and
    last rows, random ones): the same rows selected in a launch of their own give the same sets bit for bit, and
    the oracle audit on fp32 scores finds no swap beyond the rounding bound."""
    from geoweave_b200.custom_indexer import sparse_topk_indexer_inference_func

    q, kx, w = make_indexer_inputs(N, N, seed=N + k, ties=ties)
    qd, kd, wd = q.to(dev()), kx.to(dev()), w.to(dev())
    idx, _ = sparse_topk_indexer_inference_func(qd, kd, wd, None, k, 0.125, return_scores=False)
    geoweave_b200.check_status()
    assert idx.shape == (1, N, k) and idx.dtype == torch.int32
    for r0 in range(0, N, 65536):
        srt = torch.sort(idx[:, r0:r0 + 65536].long(), -1).values
        assert int(srt.min()) >= 0 and int(srt.max()) < N
        assert not bool((srt[..., 1:] == srt[..., :-1]).any())
    g = torch.Generator().manual_seed(N)
    edges = torch.tensor([0, 1, 127, 128, N // 2 - 1, N // 2, N - 129, N - 128, N - 2, N - 1])
    rows = torch.unique(torch.cat([edges, torch.randperm(N, generator=g)[:n_audit]]))
    picked = torch.sort(idx[:, rows.to(dev())].long(), -1).values.cpu()
    alone, _ = sparse_topk_indexer_inference_func(qd[:, rows.to(dev())].contiguous(), kd, wd, None, k, 0.125, return_scores=False)
    geoweave_b200.check_status()
    assert torch.equal(torch.sort(alone.long(), -1).values.cpu(), picked)
    swapped = 0
    for c0 in range(0, rows.numel(), 64):
        r = rows[c0:c0 + 64]
        scores = orc.indexer_scores(q[:, r], kx, w, 0.125, row_chunk=64)
        res = orc.audit_topk(picked[:, c0:c0 + 64], scores, k, q[:, r], kx, w, 0.125)
        assert res["out_of_range"] == 0 and res["duplicates"] == 0 and res["unexplained"] == 0, (N, c0, res)
        swapped += res["swapped"]
    assert swapped <= 0.02 * rows.numel() * k, swapped


def _device_inputs(T, S, seed, ties):
    """bf16 q_idx [1,T,4,64], k_idx [1,S,4,64] ~N(0,1), w [1,S,4] ~U(0,1), made on the device; the tie variant overwrites
    10 % of the key rows (k_idx AND w) by copies of random other rows."""
    g = torch.Generator(device=dev()).manual_seed(seed)
    q = torch.randn(1, T, 4, 64, device=dev(), generator=g).bfloat16()
    kx = torch.randn(1, S, 4, 64, device=dev(), generator=g).bfloat16()
    w = torch.rand(1, S, 4, device=dev(), generator=g).bfloat16()
    if ties:
        n_dup = S // 10
        dst = torch.randperm(S, device=dev(), generator=g)[:n_dup]
        src = torch.randint(0, S, (n_dup,), device=dev(), generator=g)
        kx[0, dst] = kx[0, src]
        w[0, dst] = w[0, src]
    return q, kx, w


@pytest.mark.parametrize("ties", [False, True])
@pytest.mark.parametrize("k", [256, 512, 1024, 2048])
@pytest.mark.parametrize("views", [8, 32, 128, 512])
def test_config5_grid_same_scores_selection_is_bit_identical(views, k, ties):
    """Every point of the sweep N = views x 1041, k in {256..2048}, with and without 10 % duplicated key rows: 256
    query rows against all N keys.  The fused kernel's selection must equal, bit for bit, the exact top-k (ties to
    the lower index) of the fp32 scores the same tensor-core main loop writes out densely."""
    from geoweave_b200.custom_indexer import sparse_topk_indexer_func
    from geoweave_b200.custom_indexer.sparse_topk_indexer import indexer_scores

    S, T = views * 1041, 256
    q, kx, w = _device_inputs(T, S, seed=views * 10000 + k + int(ties), ties=ties)
    dense = indexer_scores(q, kx, w, 0.125)
    idx, sc = sparse_topk_indexer_func(q, kx, w, None, k, 0.125, 256)
    geoweave_b200.check_status()
    order = torch.sort(dense, dim=-1, descending=True, stable=True).indices[..., :k]
    expect = torch.sort(order, dim=-1).values
    got = torch.sort(idx.long(), dim=-1).values
    assert torch.equal(got, expect), (views, k, ties, int((got != expect).any(-1).sum()))
    assert torch.equal(sc.float(), dense.gather(-1, idx.long()).bfloat16().float())
    if ties:  # the duplicates really produce ties at the boundary in some rows: the k-th and (k+1)-th score are equal
        top = torch.sort(dense, dim=-1, descending=True).values
        assert bool((top[..., k - 1] == top[..., k]).any())


def test_score_topk_fused_select_returns_the_selected_scores_and_positions():
    """The k = 512 wrapper of the reference (score_topk_fused_cuda.py:48-95), here for any k taken from the outputs."""
    from geoweave_b200.custom_indexer.score_topk_fused_cuda import is_score_topk_fused_available, score_topk_fused_select
    from geoweave_b200.custom_indexer.sparse_topk_indexer import indexer_scores

    assert is_score_topk_fused_available()
    for T, S, K, ties in ((90, 3000, None, False), (200, 9000, 1024, True)):
        q, kx, w = _device_inputs(T, S, seed=S, ties=ties)
        dense = indexer_scores(q, kx, w, 0.125)
        if K is None:
            sc, pos = score_topk_fused_select(q, kx, w, softmax_scale=0.125)
            K = 512  # the reference's fixed size
        else:
            out_pos = torch.full((1, T, K), -7, dtype=torch.int32, device=dev())
            out_sc = torch.full((1, T, K), float("nan"), dtype=torch.bfloat16, device=dev())
            sc, pos = score_topk_fused_select(q, kx, w, softmax_scale=0.125, out_scores=out_sc, out_pos=out_pos)
            assert sc.data_ptr() == out_sc.data_ptr() and pos.data_ptr() == out_pos.data_ptr()
        geoweave_b200.check_status()
        assert tuple(pos.shape) == (1, T, K) and pos.dtype == torch.int32 and sc.dtype == q.dtype
        order = torch.sort(dense, dim=-1, descending=True, stable=True).indices[..., :K]
        assert torch.equal(torch.sort(pos.long(), -1).values, torch.sort(order, -1).values)
        assert torch.equal(sc.float(), dense.gather(-1, pos.long()).bfloat16().float())


def test_indexer_and_attention_replay_from_a_cuda_graph():
    """Both operators only enqueue on the caller's stream (no allocation, no synchronisation inside the C calls), so a
    layer can be captured once and replayed on new contents of the same buffers."""
    from geoweave_b200.custom_flash_attn import sparse_index_flash_attn_inference_func
    from geoweave_b200.custom_indexer import sparse_topk_indexer_inference_func

    N, k = 8328, 256
    g = torch.Generator().manual_seed(5)

    def fresh():
        qi, ki, w = make_indexer_inputs(N, N, seed=int(torch.randint(0, 1 << 30, (1,), generator=g)))
        qkv = [torch.randn(1, N, 16, 64, generator=g).bfloat16() for _ in range(3)]
        return [x.to(dev()) for x in (qi, ki, w, *qkv)]

    def layer(qi, ki, w, q, kk, v):
        idx, _ = sparse_topk_indexer_inference_func(qi, ki, w, None, k, 0.125, return_scores=False)
        out, _ = sparse_index_flash_attn_inference_func(q, kk, v, idx, None, False, 0.125)
        return idx, out

    static = fresh()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        layer(*static)  # sizes the cached workspace outside the capture
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        idx_g, out_g = layer(*static)
    for _ in range(2):
        new = fresh()
        for dst, src in zip(static, new):
            dst.copy_(src)
        graph.replay()
        torch.cuda.synchronize()
        idx_e, out_e = layer(*new)
        geoweave_b200.check_status()
        assert torch.equal(sorted_idx(idx_g), sorted_idx(idx_e))
        assert (out_g.float() - out_e.float()).abs().max().item() <= 2e-2  # the order inside a row is not promised
