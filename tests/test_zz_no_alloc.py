"""The no-allocation score entry point (gw_indexer_scores_noalloc), called through the C ABI.

It exists for hosts that may not allocate device memory themselves -- a plugin inside a runtime that owns the
device heap, or a loop that cannot afford the synchronisation an allocation can cause.  Its scratch is a fixed
array inside the library, shared by all calls, so the checks below are: results identical to the allocating
entry point, on two calls in a row (the second smaller, so leftovers of the first would show), and a clear
refusal beyond the fixed capacity.  This file sorts last on purpose.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

NOALLOC_MAX_KEYS = 262144
GW_ERR_TOO_LARGE = -7


def _call(lib, fn, q, k, w, key_step, out):
    from geoweave_b200 import _lib

    B, T, Hi, Di = q.shape
    S = k.shape[1]
    dev = q.device
    with torch.cuda.device(dev):
        return fn(q.data_ptr(), k.data_ptr(), w.data_ptr(), _lib.dtype_code(q), B, T, S, Hi, Di, 0.125, key_step,
                  out.data_ptr(), out.shape[-1], _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev))


def test_noalloc_scores_equal_allocating_entry_on_two_calls_in_a_row():
    import geoweave_b200
    from geoweave_b200 import _lib
    from tests.gpu_util import dev, make_indexer_inputs

    lib = _lib.load()
    for call, (T, S, step, seed) in enumerate([(300, 5000, 1, 1), (130, 1041, 3, 2)]):
        q, k, w = [x.to(dev()) for x in make_indexer_inputs(T, S, seed=seed, negw=True)]
        m = (S + step - 1) // step
        expect = torch.full((1, T, m), float("nan"), device=dev())
        got = torch.full((1, T, m), float("nan"), device=dev())
        _lib.check(_call(lib, lib.gw_indexer_scores, q, k, w, step, expect), "gw_indexer_scores")
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        _lib.check(_call(lib, lib.gw_indexer_scores_noalloc, q, k, w, step, got), "gw_indexer_scores_noalloc")
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        geoweave_b200.check_status()
        assert not torch.isnan(got).any()
        assert torch.equal(got, expect), f"call {call}"  # same kernels, same table values: bit-identical


def test_noalloc_refuses_problems_beyond_its_fixed_capacity():
    from geoweave_b200 import _lib
    from tests.gpu_util import dev

    lib = _lib.load()
    S = NOALLOC_MAX_KEYS  # + tile padding exceeds the table
    q = torch.zeros(1, 1, 4, 64, dtype=torch.bfloat16, device=dev())
    k = torch.zeros(1, S, 4, 64, dtype=torch.bfloat16, device=dev())
    w = torch.zeros(1, S, 4, dtype=torch.bfloat16, device=dev())
    out = torch.zeros(1, 1, S, device=dev())
    rc = _call(lib, lib.gw_indexer_scores_noalloc, q, k, w, 1, out)
    assert rc == GW_ERR_TOO_LARGE
    assert b"capacity" in lib.gw_strerror(rc)
    with pytest.raises(_lib.GeoWeaveError):
        _lib.check(rc, "gw_indexer_scores_noalloc")
