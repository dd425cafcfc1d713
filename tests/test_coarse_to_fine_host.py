"""Host logic of the coarse-to-fine selection on CPU: the source table and the number of kept sources against fixtures
produced by the reference (``tests/golden/make_golden_c2f.py``)."""
import numpy as np
import pytest

from geoweave_b200.coarse_to_fine import source_layout
from tests import golden
from tests.golden.make_golden_c2f import CASES

GOLD = golden.load("reference_c2f.npz")


@pytest.mark.parametrize("name", sorted(CASES))
def test_source_table_and_budget_match_the_reference(name):
    tpv, views, special, gh, gw, topk, _, _ = CASES[name]
    lay = source_layout(tpv, views, special, gh, gw, "cpu")
    g = GOLD[name]
    assert np.array_equal(lay.table.numpy(), g["table"])
    assert [lay.source_len, lay.special_count, lay.edge_count, lay.coarse_count] == g["counts"][:4].tolist()
    assert lay.kept_sources(topk) == int(g["counts"][4])
    if "fine_to_row" in g:
        assert np.array_equal(lay.token_source.numpy(), g["fine_to_row"])
    assert source_layout(tpv, views, special, gh, gw, "cpu") is lay  # cached


def test_a_grid_that_does_not_match_is_refused():
    with pytest.raises(ValueError):
        source_layout(100, 2, 5, 10, 10, "cpu")
