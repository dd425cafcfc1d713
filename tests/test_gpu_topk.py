"""GPU parity: exact top-k of materialised scores and the merge of two lists, through the C ABI."""
import pytest
import torch

from oracle import gw_oracle as orc
from tests.gpu_util import dev, sorted_idx, t

pytestmark = pytest.mark.gpu

IDX_CASES = ["idx_int", "idx_int_ties", "idx_bf16", "idx_bf16_ties", "idx_negw", "idx_kgeS", "idx_h2d32"]


@pytest.mark.parametrize("name", IDX_CASES)
def test_topk_exact_on_reference_scores_is_bit_identical(golden, name):
    from geoweave_b200.custom_indexer.topk_exact_cuda import topk_exact_select

    c = golden[name]
    sc = t(c["scores"])
    k = min(int(c["k"]), sc.shape[-1])
    vals, pos = topk_exact_select(sc, k=k)
    assert pos.dtype == torch.int64 and vals.dtype == sc.dtype
    assert torch.equal(sorted_idx(pos), torch.from_numpy(c["tie_idx"]).long())
    assert torch.equal(vals.cpu(), torch.from_numpy(c["scores"]).gather(-1, pos.cpu()))


@pytest.mark.parametrize("cols,k", [(4164, 1024), (8328, 256), (33312, 1024), (33312, 2048), (133248, 512), (1000, 1000), (700, 1)])
@pytest.mark.parametrize("kind", ["randn", "ties", "const"])
def test_topk_exact_sweep(cols, k, kind):
    from geoweave_b200.custom_indexer.topk_exact_cuda import topk_exact_select

    g = torch.Generator().manual_seed(cols + k)
    rows = 6
    if kind == "randn":
        sc = torch.randn(1, rows, cols, generator=g)
    elif kind == "ties":
        sc = torch.randint(0, 50, (1, rows, cols), generator=g).float() * 0.25 - 3.0
        sc[0, 0, ::3] = -0.0
        sc[0, 0, 1::3] = 0.0
    else:
        sc = torch.full((1, rows, cols), 0.5)
    out_pos = torch.empty((1, rows, k), dtype=torch.int32, device=dev())
    vals, pos = topk_exact_select(sc.to(dev()), out_pos=out_pos)
    assert torch.equal(sorted_idx(pos), orc.topk_tie_exact(sc, k).long())


@pytest.mark.parametrize("cols,k,rows", [(8328, 256, 1300), (8329, 512, 40), (33312, 1024, 300), (40001, 64, 10), (60000, 1024, 5)])
@pytest.mark.parametrize("kind", ["heavy_tail", "narrow", "mostly_zero"])
def test_topk_exact_many_rows_and_awkward_distributions(cols, k, rows, kind):
    """Rows in shared memory (CTAs walk several rows; odd widths take plain loads; 60000 columns do not fit and go
    to the re-reading kernel), with score distributions that defeat a sampled threshold or crowd the boundary."""
    from geoweave_b200.custom_indexer.topk_exact_cuda import topk_exact_select

    g = torch.Generator().manual_seed(cols * 3 + k)
    if kind == "heavy_tail":
        sc = torch.exp(3.0 * torch.randn(1, rows, cols, generator=g)) * torch.sign(torch.randn(1, rows, cols, generator=g))
    elif kind == "narrow":
        sc = 1.0 + torch.randint(0, 4096, (1, rows, cols), generator=g).float() * 2.0 ** -20
    else:
        sc = torch.relu(torch.randn(1, rows, cols, generator=g) - 2.2)  # about 1.4 % of the columns are positive
    vals, pos = topk_exact_select(sc.to(dev()), k=k)
    assert torch.equal(sorted_idx(pos), orc.topk_tie_exact(sc, k).long())
    assert torch.equal(vals.cpu(), sc.gather(-1, pos.cpu()))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_topk_exact_16bit_scores(dtype):
    from geoweave_b200.custom_indexer.topk_exact_cuda import topk_exact_select

    g = torch.Generator().manual_seed(1)
    sc = torch.randn(2, 5, 3000, generator=g).to(dtype)  # 16-bit scores tie a lot
    vals, pos = topk_exact_select(sc.to(dev()), k=512)
    assert torch.equal(sorted_idx(pos), orc.topk_tie_exact(sc.float(), 512).long())
    assert torch.equal(vals.cpu(), sc.gather(-1, pos.cpu()))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("cols,k", [(16384, 512), (33312, 1024)])
def test_topk_exact_16bit_scores_on_the_sampled_path(dtype, cols, k):
    """Wide 16-bit rows: plain loads into shared memory, sampled threshold, and boundaries crowded with equal values."""
    from geoweave_b200.custom_indexer.topk_exact_cuda import topk_exact_select

    g = torch.Generator().manual_seed(cols + k)
    sc = (torch.randn(1, 40, cols, generator=g) * 2.0).to(dtype)
    vals, pos = topk_exact_select(sc.to(dev()), k=k)
    assert torch.equal(sorted_idx(pos), orc.topk_tie_exact(sc.float(), k).long())
    assert torch.equal(vals.cpu(), sc.gather(-1, pos.cpu()))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_merge_two_topk_16bit_scores(dtype):
    from geoweave_b200.custom_indexer.merge_two_topk_cuda import merge_two_topk_inplace

    g = torch.Generator().manual_seed(17)
    rows, k, start = 33, 1024, 20000
    a_s = torch.randn(1, rows, k, generator=g).to(dtype)
    b_s = torch.randn(1, rows, k, generator=g).to(dtype)
    a_i = torch.stack([torch.randperm(start, generator=g)[:k] for _ in range(rows)]).view(1, rows, k).to(torch.int32)
    b_p = torch.stack([torch.randperm(9000, generator=g)[:k] for _ in range(rows)]).view(1, rows, k)
    exp_s, exp_i = orc.merge_two_topk(a_s.float(), a_i, b_s.float(), b_p + start, k)
    o_s, o_i = torch.empty_like(a_s, device=dev()), torch.empty_like(a_i, device=dev())
    assert merge_two_topk_inplace(a_s.to(dev()), a_i.to(dev()), b_s.to(dev()), b_p.to(dev()), start, o_s, o_i) is True
    order = torch.sort(o_i.long(), -1)
    assert torch.equal(order.values.cpu(), exp_i.long())
    assert torch.equal(o_s.gather(-1, order.indices).float().cpu(), exp_s)


def test_topk_exact_rejects_short_rows():
    from geoweave_b200.custom_indexer.topk_exact_cuda import topk_exact_select

    with pytest.raises(ValueError):
        topk_exact_select(torch.zeros(1, 2, 100, device=dev()))  # default K = 512 as in the reference


@pytest.mark.parametrize("k,kb", [(512, 512), (1024, 256), (64, 64), (2048, 2048)])
def test_merge_two_topk_matches_oracle(k, kb):
    from geoweave_b200.custom_indexer.merge_two_topk_cuda import merge_two_topk_inplace

    g = torch.Generator().manual_seed(k * 7 + kb)
    rows, start = 9, 5000
    a_s = torch.randint(0, 40, (1, rows, k), generator=g).float() / 4
    b_s = torch.randint(0, 40, (1, rows, kb), generator=g).float() / 4
    a_i = torch.stack([torch.randperm(start, generator=g)[:k] for _ in range(rows)]).view(1, rows, k).to(torch.int32)
    b_p = torch.stack([torch.randperm(3000, generator=g)[:kb] for _ in range(rows)]).view(1, rows, kb)
    exp_s, exp_i = orc.merge_two_topk(a_s, a_i, b_s, b_p + start, k)
    A_s, A_i = a_s.to(dev()), a_i.to(dev())
    ok = merge_two_topk_inplace(A_s, A_i, b_s.to(dev()), b_p.to(dev()), start, A_s, A_i)  # in place, as the reference uses it
    assert ok is True
    order = torch.sort(A_i.long(), -1)
    assert torch.equal(order.values.cpu(), exp_i.long())
    assert torch.equal(A_s.gather(-1, order.indices).cpu(), exp_s)


def test_merge_two_topk_reports_failure_like_the_reference():
    from geoweave_b200.custom_indexer.merge_two_topk_cuda import merge_two_topk_inplace

    z = torch.zeros(1, 1, 4, device=dev())
    zi = torch.zeros(1, 1, 4, dtype=torch.int32, device=dev())
    assert merge_two_topk_inplace(z, zi, z, zi, 0, z, zi) is False  # pending_pos must be int64
