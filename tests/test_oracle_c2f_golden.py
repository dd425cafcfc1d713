"""The oracle's restatement of the reference's coarse-to-fine selector pieces against fixtures produced by the
reference itself (``tests/golden/make_golden_c2f.py``): source layout, number of sources kept, pooled keys and weights,
expansion of ordered source lists to token indices."""
import numpy as np
import pytest
import torch

from oracle import gw_oracle as orc
from tests import golden
from tests.golden.make_golden_c2f import CASES

GOLD = golden.load("reference_c2f.npz")


@pytest.mark.parametrize("name", sorted(CASES))
def test_layout_and_kept_sources(name):
    tpv, views, special, gh, gw, topk, _, _ = CASES[name]
    lay = orc.source_layout(tpv, views, special, gh, gw)
    g = GOLD[name]
    assert np.array_equal(lay["source_to_fine"].numpy(), g["table"])
    assert [lay["source_len"], lay["special_count"], lay["edge_count"], lay["coarse_count"]] == g["counts"][:4].tolist()
    assert orc.coarse_topk(lay, topk) == int(g["counts"][4])


@pytest.mark.parametrize("name", [n for n in sorted(CASES) if CASES[n][7]])
def test_pooled_sources(name):
    tpv, views, special, gh, gw, _, _, _ = CASES[name]
    lay = orc.source_layout(tpv, views, special, gh, gw)
    g = GOLD[name]
    ks, ws = orc.pool_sources(torch.from_numpy(g["k"]), torch.from_numpy(g["w"]), lay)
    assert np.allclose(ks.numpy(), g["src_k"], rtol=0, atol=1e-6)
    assert np.allclose(ws.numpy(), g["src_w"], rtol=0, atol=1e-6)
    # pooled queries (the whole sequence as one chunk) are the same means, and every token takes its source's row
    assert np.allclose(ks.numpy(), g["coarse_q"], rtol=0, atol=1e-6)
    assert np.array_equal(orc.token_source(lay).numpy(), g["fine_to_row"])


@pytest.mark.parametrize("name", sorted(CASES))
def test_expansion_of_ordered_lists(name):
    tpv, views, special, gh, gw, topk, _, _ = CASES[name]
    lay = orc.source_layout(tpv, views, special, gh, gw)
    g = GOLD[name]
    fine = orc.expand_sources(torch.from_numpy(g["lists"]), lay, topk, tpv * views)
    assert np.array_equal(fine.numpy(), g["fine"])
