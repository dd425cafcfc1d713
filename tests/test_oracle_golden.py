"""Pin the CPU oracle to outputs of the reference's own CPU code (tests/golden/reference_cpu.npz)."""
import numpy as np
import pytest
import torch

from oracle import gw_oracle as orc

IDX_CASES = ["idx_int", "idx_int_ties", "idx_bf16", "idx_bf16_ties", "idx_negw", "idx_kgeS", "idx_h2d32"]
ATTN_CASES = ["attn_h4", "attn_h16", "attn_tnes", "attn_d128", "attn_d32"]


def _t(x):
    return torch.from_numpy(np.ascontiguousarray(x))


@pytest.mark.parametrize("name", IDX_CASES)
def test_scores_match_reference(golden, name):
    c = golden[name]
    sc = orc.indexer_scores(_t(c["q_idx"]), _t(c["k_idx"]), _t(c["w"]), float(c["scale"]))
    ref = _t(c["scores"])
    if name.startswith("idx_int"):
        # integer inputs and dyadic weights: every product and partial sum is exact in fp32
        assert torch.equal(sc, ref)
    else:
        torch.testing.assert_close(sc, ref, rtol=0, atol=2e-6 * float(ref.abs().max()))


@pytest.mark.parametrize("name", IDX_CASES)
def test_topk_tie_exact_matches_stable_sort_of_reference_scores(golden, name):
    c = golden[name]
    idx = orc.topk_tie_exact(_t(c["scores"]), int(c["k"]))
    assert torch.equal(idx, _t(c["tie_idx"]))


@pytest.mark.parametrize("name", IDX_CASES)
def test_topk_is_a_valid_answer_for_the_reference(golden, name):
    """The reference's torch.topk and its block-wise CPU op leave tie order open: as VALUE multisets all agree."""
    c = golden[name]
    sc = _t(c["scores"])
    mine = orc.topk_tie_exact(sc, int(c["k"])).long()
    for key in ("ref_idx", "blk_idx"):
        theirs = _t(c[key]).long()
        a = torch.sort(sc.gather(-1, mine), -1).values
        b = torch.sort(sc.gather(-1, theirs), -1).values
        assert torch.equal(a, b), key
        # and wherever a row has no tie at its k-th value the index sets are identical
        kth = a[..., :1]
        tie_rows = ((sc == kth).sum(-1) > 1)
        same = (torch.sort(theirs, -1).values == mine).all(-1)
        assert bool((same | tie_rows).all()), key


def test_end_to_end_indexer_topk_on_exact_inputs(golden):
    for name in ("idx_int", "idx_int_ties"):
        c = golden[name]
        idx, sc = orc.indexer_topk(_t(c["q_idx"]), _t(c["k_idx"]), _t(c["w"]), int(c["k"]), float(c["scale"]))
        assert torch.equal(idx, _t(c["tie_idx"]))
        assert torch.equal(sc, _t(c["scores"]).gather(-1, idx.long()))


def test_audit_accepts_reference_topk_only_as_ties(golden):
    c = golden["idx_int_ties"]
    res = orc.audit_topk(_t(c["ref_idx"]), _t(c["scores"]), int(c["k"]))
    assert res["unexplained"] == 0 and res["swapped"] > 0 and res["max_gap"] == 0.0
    bad = _t(c["tie_idx"]).clone()
    sc = _t(c["scores"])[0, 0]
    worst = int(torch.argmin(sc))
    if worst not in bad[0, 0].tolist():
        bad[0, 0, 0] = worst
        res = orc.audit_topk(bad, _t(c["scores"]), int(c["k"]))
        assert res["unexplained"] >= 1


@pytest.mark.parametrize("name", ATTN_CASES)
def test_sparse_attention_matches_reference(golden, name):
    c = golden[name]
    out, lse, asum = orc.sparse_attention(_t(c["q"]), _t(c["k"]), _t(c["v"]), _t(c["idx"]), float(c["scale"]))
    torch.testing.assert_close(out, _t(c["out"]), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(asum, _t(c["attn_sum"]), rtol=1e-5, atol=1e-5)
    assert torch.isfinite(lse).all()
    if "idx_pad" in c:
        out, lse, asum = orc.sparse_attention(_t(c["q"]), _t(c["k"]), _t(c["v"]), _t(c["idx_pad"]), float(c["scale"]))
        torch.testing.assert_close(out, _t(c["out_pad"]), rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(asum, _t(c["attn_sum_pad"]), rtol=1e-5, atol=1e-5)


def test_sparse_attention_padding_rules():
    g = torch.Generator().manual_seed(3)
    q = torch.randn(1, 3, 2, 8, generator=g)
    k = torch.randn(1, 5, 2, 8, generator=g)
    v = torch.randn(1, 5, 2, 8, generator=g)
    idx = torch.tensor([[[0, 1, -1, 7], [4, 4, 2, 5], [-1, -1, 9, -3]]], dtype=torch.int32)
    out, lse, asum = orc.sparse_attention(q, k, v, idx)
    assert torch.equal(out[0, 2], torch.zeros(2, 8)) and bool(torch.isinf(lse[0, :, 2]).all())
    assert float(asum[0, 0, 2]) == 0.0 and float(asum[0, 0, 3]) == 0.0  # -1 and >= S are padding
    torch.testing.assert_close(asum[0, :2].sum(-1), torch.full((2,), 2.0))  # two heads, each row of p sums to 1
    assert float(asum[0, 1, 0]) == float(asum[0, 1, 1])  # a key listed twice counts twice


def test_merge_two_topk_equals_topk_of_union():
    g = torch.Generator().manual_seed(5)
    S, k = 64, 8
    sc = torch.randint(0, 6, (4, S), generator=g).float()  # many ties
    left, right = sc[:, :40], sc[:, 40:]
    a_i = orc.topk_tie_exact(left, k)
    b_i = orc.topk_tie_exact(right, k) + 40
    m_s, m_i = orc.merge_two_topk(sc.gather(-1, a_i.long()), a_i, sc.gather(-1, b_i.long()), b_i, k)
    assert torch.equal(m_i, orc.topk_tie_exact(sc, k))
    assert torch.equal(m_s, sc.gather(-1, m_i.long()))


@pytest.mark.parametrize("name", ["fe_f32", "fe_bf16", "fe_pi3_bf16"])
def test_front_end_restatement_matches_the_reference_modules(name):
    """q/k LayerNorm + rotary embedding, v, and the indexer's projections after the fused linear layer
    (fixtures from DSAAttention / LightningIndexer / RotaryPositionEmbedding2D run on CPU)."""
    import numpy as np

    from tests import golden as golden_pkg

    c = golden_pkg.load("reference_frontend.npz")[name]
    T = lambda a: torch.from_numpy(np.asarray(a))
    outs = orc.project_front_end(T(c["fused"]), T(c["pos"]), T(c["cos"]), T(c["sin"]), int(c["heads"]), 64, 4, 64,
                                 (T(c["q_norm_w"]), T(c["q_norm_b"]), float(c["eps"])),
                                 (T(c["k_norm_w"]), T(c["k_norm_b"]), float(c["eps"])),
                                 (T(c["ik_norm_w"]), T(c["ik_norm_b"]), float(c["ik_norm_eps"])))
    exact = name == "fe_f32"
    for nm, o in zip(["q", "k", "v", "q_idx", "k_idx", "w"], outs):
        ref = T(c[nm])
        err = (o - ref).abs()
        # fp32 modules: rounding order only; bf16 modules round after every operation (two units in the last place)
        tol = 2e-5 + 2e-6 * ref.abs() if exact else 2e-2 + 2.0 ** -7 * ref.abs()
        assert bool((err <= tol).all()), (nm, float(err.max()))
    # the linear layer itself: x @ weight^T + bias reproduces the recorded output
    lin = torch.nn.functional.linear(T(c["x"]), T(c["weight"]), T(c["bias"]))
    assert (lin - T(c["fused"])).abs().max().item() <= (1e-4 if exact else 6e-2)


def test_rope_tables_follow_the_reference_rounding():
    import numpy as np

    from geoweave_b200.front_end import rope_tables
    from tests import golden as golden_pkg

    G = golden_pkg.load("reference_frontend.npz")
    for name, dtype in (("fe_f32", torch.float32), ("fe_bf16", torch.bfloat16)):
        c = G[name]
        cos, sin = rope_tables(c["cos"].shape[0], "cpu", dtype)
        assert torch.equal(cos, torch.from_numpy(np.asarray(c["cos"]))) and torch.equal(sin, torch.from_numpy(np.asarray(c["sin"])))
