"""The peer-memory exchange on ONE GPU (a group of one rank): pack, flag barrier, pull by kernel and by copies run and
give back the rows they were given, for aligned and unaligned row sizes, twice in a row (both buffer halves) and after
the buffers had to grow.  The multi-rank behaviour is checked by ``bench.py --gpus N`` itself, which compares the
exchange with the NCCL all-gather before it times anything."""
import pytest
import torch
import torch.distributed as dist

import geoweave_b200
from tests.gpu_util import dev

pytestmark = pytest.mark.gpu


@pytest.fixture()
def one_rank_group():
    if dist.is_initialized():
        yield dist.group.WORLD
        return
    torch.cuda.set_device(dev())
    dist.init_process_group("nccl", init_method="tcp://127.0.0.1:29631", rank=0, world_size=1, device_id=dev())
    try:
        yield dist.group.WORLD
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
@pytest.mark.parametrize("pull", ["kernel", "copies"])
def test_exchange_of_one_rank_returns_the_rows(one_rank_group, pull):
    from geoweave_b200.sharding import PeerExchange

    try:
        ex = PeerExchange(group=one_rank_group, device=dev(), pull=pull, copy_streams=3, limit_ms=500)
    except Exception as exc:  # peer-mapped memory is not available in every environment
        pytest.skip(f"symmetric memory could not be set up: {type(exc).__name__}: {exc}")
    g = torch.Generator().manual_seed(0)
    for rows in (257, 1001, 40000):  # the last one makes the buffers grow
        k_idx = torch.randn(1, rows, 4, 64, generator=g).bfloat16().to(dev())
        w = torch.randn(1, rows, 3, generator=g).bfloat16().to(dev())     # 6-byte rows: the unaligned path
        f = torch.randn(1, rows, 5, generator=g).to(dev())
        for rep in range(3):
            outs = ex.gather([k_idx, w, f], rows, async_op=(rep == 1)).result()
            torch.cuda.synchronize()
            assert all(torch.equal(a, b) and a.data_ptr() != b.data_ptr() for a, b in zip(outs, (k_idx, w, f)))
    geoweave_b200.check_status()
    with pytest.raises(ValueError):
        ex.gather([k_idx[:, :10]], rows)


def test_barrier_wait_runs_out_when_a_peer_never_signals():
    """Two flag arrays on this GPU stand for two ranks; nobody plays rank 1, so rank 0's wait for it must end after the
    given limit with GW_ERR_TIMEOUT in the status word -- and the context stays usable."""
    import time

    from geoweave_b200 import _lib

    lib = _lib.load()
    flags = torch.zeros(2, 64, dtype=torch.int32, device=dev())
    ptrs = torch.tensor([flags[0].data_ptr(), flags[1].data_ptr()], dtype=torch.int64, device=dev())
    status = _lib.status_word(dev())
    status.zero_()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    with torch.cuda.device(dev()):
        rc = lib.gw_peer_barrier(ptrs.data_ptr(), 0, 2, 1, 20, status.data_ptr(), _lib.stream_ptr(dev()))
    assert rc == 0
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert 0.015 <= waited < 1.0, waited
    assert int(status.item()) == _lib.GW_ERR_TIMEOUT
    assert flags[0, 0].item() == 1 and flags[1, 0].item() == 1 and flags[0, 1].item() == 0  # rank 0 signalled both, rank 1 never did
    with pytest.raises(_lib.GeoWeaveError):
        geoweave_b200.check_status()
    status.zero_()
    # a barrier whose peers have all arrived (the flags are already there) passes at once
    flags[0, 1] = 1
    with torch.cuda.device(dev()):
        assert lib.gw_peer_barrier(ptrs.data_ptr(), 0, 2, 1, 20, status.data_ptr(), _lib.stream_ptr(dev())) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    geoweave_b200.check_status()
