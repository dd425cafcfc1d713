"""Device-side failure reporting: a wait that cannot be satisfied ends after its limit, the kernel records
GW_ERR_TIMEOUT in the status word and returns, `check_status()` raises, and the context goes on working.

The wait that runs out here is in a one-warp diagnostic kernel made for this purpose (a barrier that nobody
signals, limit of a few milliseconds); it uses the same bounded-wait routine as every pipeline of the library.
Nothing faults, traps or hangs."""
import pytest
import torch

pytestmark = pytest.mark.gpu

GW_ERR_TIMEOUT = -5


def test_a_wait_that_runs_out_sets_the_status_word_and_the_next_call_is_correct():
    import geoweave_b200
    from geoweave_b200 import _lib
    from geoweave_b200.custom_indexer import sparse_topk_indexer_func
    from oracle import gw_oracle as orc
    from tests.gpu_util import dev, make_indexer_inputs, sorted_idx

    lib = _lib.load()
    geoweave_b200.check_status()  # start from a clean status word
    status = _lib.status_word(dev())
    waited = torch.zeros(1, dtype=torch.int64, device=dev())
    limit_us = 3000
    with torch.cuda.device(dev()):
        rc = lib.gw_debug_bounded_wait_selftest(limit_us, status.data_ptr(), waited.data_ptr(), _lib.stream_ptr(dev()))
    _lib.check(rc, "gw_debug_bounded_wait_selftest")
    torch.cuda.synchronize()  # returns: the kernel ended by itself
    ns = int(waited.item())
    assert limit_us * 1000 <= ns < 200 * limit_us * 1000, ns  # it waited for its limit, not for ever
    assert int(status.item()) == GW_ERR_TIMEOUT
    with pytest.raises(_lib.GeoWeaveError) as err:
        geoweave_b200.check_status()
    assert err.value.code == GW_ERR_TIMEOUT and "bounded wait" in str(err.value)
    geoweave_b200.check_status()  # reading the status cleared it
    # the context is intact: the next call of the real path is exact
    q, k, w = make_indexer_inputs(200, 900, seed=5, integer=True)
    idx, _ = sparse_topk_indexer_func(q.to(dev()), k.to(dev()), w.to(dev()), None, 64, 0.125, 256)
    geoweave_b200.check_status()
    ref, _ = orc.indexer_topk(q, k, w, 64, 0.125)
    assert torch.equal(sorted_idx(idx), ref.long())


def test_selftest_arguments_are_checked_on_the_host():
    from geoweave_b200 import _lib
    from tests.gpu_util import dev

    lib = _lib.load()
    status = _lib.status_word(dev())
    assert lib.gw_debug_bounded_wait_selftest(0, status.data_ptr(), None, None) == -1
    assert lib.gw_debug_bounded_wait_selftest(10 ** 6, status.data_ptr(), None, None) == -1  # more than 0.1 s is refused
    assert lib.gw_debug_bounded_wait_selftest(100, None, None, None) == -1


def test_device_cache_reset_is_harmless_between_calls():
    import geoweave_b200
    from geoweave_b200 import _lib
    from geoweave_b200.custom_indexer import sparse_topk_indexer_func
    from oracle import gw_oracle as orc
    from tests.gpu_util import dev, make_indexer_inputs, sorted_idx

    lib = _lib.load()
    q, k, w = make_indexer_inputs(150, 700, seed=6, integer=True)
    ref, _ = orc.indexer_topk(q, k, w, 32, 0.125)
    for _ in range(2):
        idx, _ = sparse_topk_indexer_func(q.to(dev()), k.to(dev()), w.to(dev()), None, 32, 0.125, 256)
        geoweave_b200.check_status()
        assert torch.equal(sorted_idx(idx), ref.long())
        assert lib.gw_device_cache_reset() == 0
