"""The no-allocation score entry point (gw_indexer_scores_noalloc), called through the C ABI.

It exists for hosts that may not allocate device memory themselves -- a plugin inside a runtime that owns the
device heap, or a loop that cannot afford the synchronisation an allocation can cause.  Its scratch is a fixed
array inside the library, shared by all calls, so the checks below are: results identical to the allocating
entry point, on two calls in a row (the second smaller, so leftovers of the first would show), with two
batches (the table is rewritten per batch), at the largest size the fixed array takes, a clear refusal beyond
it -- and that the call really leaves the device's memory pool alone, read from the driver's own counters
(torch's allocator statistics cannot see an allocation made inside the library).  This file sorts last on purpose.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

NOALLOC_MAX_KEYS = 262144
GW_ERR_TOO_LARGE = -7

# CUmemPool_attribute values of the CUDA driver API
_RESERVED_MEM_HIGH, _USED_MEM_HIGH = 6, 8


class _DefaultPool:
    """High-water marks of the current device's default stream-ordered memory pool, through libcuda.  Every
    cudaMallocAsync in the process -- also one made by a statically linked runtime inside a library -- is served
    from this pool and raises `used high`."""

    def __init__(self, device_index: int):
        self.cu = ctypes.CDLL("libcuda.so.1")
        dev = ctypes.c_int()
        assert self.cu.cuDeviceGet(ctypes.byref(dev), device_index) == 0
        self.pool = ctypes.c_void_p()
        assert self.cu.cuDeviceGetDefaultMemPool(ctypes.byref(self.pool), dev) == 0

    def reset(self):
        zero = ctypes.c_uint64(0)
        for attr in (_RESERVED_MEM_HIGH, _USED_MEM_HIGH):
            assert self.cu.cuMemPoolSetAttribute(self.pool, attr, ctypes.byref(zero)) == 0

    def highs(self):
        out = []
        for attr in (_RESERVED_MEM_HIGH, _USED_MEM_HIGH):
            v = ctypes.c_uint64(0)
            assert self.cu.cuMemPoolGetAttribute(self.pool, attr, ctypes.byref(v)) == 0
            out.append(int(v.value))
        return tuple(out)


def _call(lib, fn, q, k, w, key_step, out):
    from geoweave_b200 import _lib

    B, T, Hi, Di = q.shape
    S = k.shape[1]
    dev = q.device
    with torch.cuda.device(dev):
        return fn(q.data_ptr(), k.data_ptr(), w.data_ptr(), _lib.dtype_code(q), B, T, S, Hi, Di, 0.125, key_step,
                  out.data_ptr(), out.shape[-1], _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev))


def _batched_inputs(B, T, S, seed):
    from tests.gpu_util import dev, make_indexer_inputs

    parts = [make_indexer_inputs(T, S, seed=seed + 17 * b, negw=True) for b in range(B)]
    return [torch.cat([p[i] for p in parts], 0).to(dev()) for i in range(3)]


def test_noalloc_scores_equal_allocating_entry_on_two_calls_in_a_row():
    import geoweave_b200
    from geoweave_b200 import _lib
    from tests.gpu_util import dev

    lib = _lib.load()
    pool = _DefaultPool(dev().index or 0)
    # (batches, rows, keys, key step): the second call is smaller than the first, the third has two batches
    for call, (B, T, S, step, seed) in enumerate([(1, 300, 5000, 1, 1), (1, 130, 1041, 3, 2), (2, 70, 2100, 2, 3)]):
        q, k, w = _batched_inputs(B, T, S, seed)
        m = (S + step - 1) // step
        expect = torch.full((B, T, m), float("nan"), device=dev())
        got = torch.full((B, T, m), float("nan"), device=dev())
        torch.cuda.synchronize()
        pool.reset()
        base = pool.highs()
        _lib.check(_call(lib, lib.gw_indexer_scores_noalloc, q, k, w, step, got), "gw_indexer_scores_noalloc")
        torch.cuda.synchronize()
        assert pool.highs() == base, "the no-allocation entry point took memory from the device's pool"
        _lib.check(_call(lib, lib.gw_indexer_scores, q, k, w, step, expect), "gw_indexer_scores")
        torch.cuda.synchronize()
        assert pool.highs()[1] > base[1], "the probe must see the allocating entry point's scratch"
        geoweave_b200.check_status()
        assert not torch.isnan(got).any()
        assert torch.equal(got, expect), f"call {call}"  # same kernels, same table values: bit-identical


def test_noalloc_takes_the_largest_size_its_array_holds():
    import geoweave_b200
    from geoweave_b200 import _lib
    from tests.gpu_util import dev

    lib = _lib.load()
    S, T = NOALLOC_MAX_KEYS - 128, 5  # round_up(S, 64) + 64 * key_step + 64 == the capacity exactly
    g = torch.Generator().manual_seed(11)
    q = torch.randn(1, T, 4, 64, generator=g).bfloat16().to(dev())
    k = torch.randn(1, S, 4, 64, generator=g).bfloat16().to(dev())
    w = torch.randn(1, S, 4, generator=g).bfloat16().to(dev())
    expect = torch.full((1, T, S), float("nan"), device=dev())
    got = torch.full((1, T, S), float("nan"), device=dev())
    _lib.check(_call(lib, lib.gw_indexer_scores_noalloc, q, k, w, 1, got), "gw_indexer_scores_noalloc")
    _lib.check(_call(lib, lib.gw_indexer_scores, q, k, w, 1, expect), "gw_indexer_scores")
    torch.cuda.synchronize()
    geoweave_b200.check_status()
    assert not torch.isnan(got).any()
    assert torch.equal(got[..., -256:], expect[..., -256:])  # the last table entries are in bounds and current
    assert torch.equal(got, expect)
    # one more key needs one more tile of table: refused
    k2 = torch.zeros(1, S + 1, 4, 64, dtype=torch.bfloat16, device=dev())
    w2 = torch.zeros(1, S + 1, 4, dtype=torch.bfloat16, device=dev())
    out2 = torch.zeros(1, T, S + 1, device=dev())
    assert _call(lib, lib.gw_indexer_scores_noalloc, q, k2, w2, 1, out2) == GW_ERR_TOO_LARGE


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
