"""Multi-rank bookkeeping of the path on CPU: world_size-2/3 gloo process groups, oracle ops as stand-ins."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from geoweave_b200.sharding import (gather_rows, gather_rows_group, gather_rows_packed, row_partition, shard_rows,
                                    sparse_global_attention_sharded)


def test_row_partition_covers_everything_once():
    for n in (0, 1, 7, 4164, 33312, 266496):
        for p in (1, 2, 3, 4, 8):
            parts = row_partition(n, p)
            assert parts[0][0] == 0 and parts[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
            sizes = [b - a for a, b in parts]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        row_partition(5, 0)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_ops():
    from oracle import gw_oracle as orc

    def indexer(qi, ki, w, k, sc):
        return orc.indexer_topk(qi, ki, w, k, sc)[0]

    def attention(q, k, v, pos, sc):
        return orc.sparse_attention(q, k, v, pos, sc)[0]

    return indexer, attention


def _worker(rank, world, port, n_tokens, case, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(123)
        full = dict(q_idx=torch.randint(-3, 4, (1, n_tokens, 2, 8), generator=g).float(),
                    k_idx=torch.randint(-3, 4, (1, n_tokens, 2, 8), generator=g).float(),
                    w=torch.randint(0, 9, (1, n_tokens, 2), generator=g).float() / 8,
                    q=torch.randn(1, n_tokens, 2, 8, generator=g), k=torch.randn(1, n_tokens, 2, 8, generator=g),
                    v=torch.randn(1, n_tokens, 2, 8, generator=g))
        mine = {n: shard_rows(x, rank, world).contiguous() for n, x in full.items()}
        if case == "roundtrip":
            for n, x in full.items():
                assert torch.equal(gather_rows(mine[n], n_tokens), x), n
            # several tensors in one collective: views of one gathered buffer, values unchanged
            ki, ww = gather_rows_packed([mine["k_idx"], mine["w"]], n_tokens).result()
            kk, vv = gather_rows_packed([mine["k"], mine["v"]], n_tokens, async_op=True).result()
            assert torch.equal(ki, full["k_idx"]) and torch.equal(ww, full["w"]) and ki.shape == full["k_idx"].shape
            assert torch.equal(kk, full["k"]) and torch.equal(vv, full["v"]) and kk.stride(-1) == 1
            # the group form (one exchange step, separate results); tensors of different dtypes are gathered one by one
            ki, ww = gather_rows_group([mine["k_idx"], mine["w"]], n_tokens).result()
            kk, vv = gather_rows_group([mine["k"], mine["v"].double()], n_tokens, async_op=True).result()
            assert torch.equal(ki, full["k_idx"]) and torch.equal(ww, full["w"])
            assert torch.equal(kk, full["k"]) and torch.equal(vv, full["v"].double()) and vv.dtype == torch.float64
            q.put((rank, "ok"))
        elif case in ("layer", "layer_exchange"):
            exchange = None
            if case == "layer_exchange":
                # stand-ins with the interface of PeerExchange (gather(xs, n_rows, async_op) -> .result()): the layer must
                # route K_idx with w through the first and K with V, asynchronously, through the second
                class Stub:
                    def __init__(self):
                        self.calls = []

                    def gather(self, xs, n_rows, async_op=False):
                        self.calls.append((len(xs), async_op))
                        return gather_rows_group(xs, n_rows, None, async_op)

                exchange = (Stub(), Stub())
            out, idx = sparse_global_attention_sharded(mine["q_idx"], mine["k_idx"], mine["w"], mine["q"], mine["k"],
                                                       mine["v"], 5, n_tokens, idx_scale=0.5, attn_scale=0.5, ops=_oracle_ops(),
                                                       exchange=exchange)
            if exchange is not None:
                assert exchange[0].calls == [(2, False)] and exchange[1].calls == [(2, True)]
            q.put((rank, (out, idx)))
        elif case == "bad_shard":
            try:
                gather_rows(mine["q"][:, :-1] if rank == 0 else mine["q"], n_tokens)
            except ValueError as exc:
                q.put((rank, f"raised: {exc}"))
            else:
                q.put((rank, "no error"))
    finally:
        dist.destroy_process_group()


def _run(world, n_tokens, case):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n_tokens, case, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in procs if True) if case != "bad_shard" else None
    if case == "bad_shard":
        results = dict([q.get(timeout=120)])
    for p in procs:
        p.join(timeout=60)
        if p.is_alive():
            p.kill()
    return results


@pytest.mark.parametrize("world,n_tokens", [(2, 10), (3, 11)])
def test_gather_rows_roundtrip_even_and_ragged(world, n_tokens):
    res = _run(world, n_tokens, "roundtrip")
    assert res == {r: "ok" for r in range(world)}


@pytest.mark.parametrize("case", ["layer", "layer_exchange"])
def test_sharded_layer_equals_single_rank_result(case):
    from oracle import gw_oracle as orc

    world, n_tokens = 2, 13
    res = _run(world, n_tokens, case)
    g = torch.Generator().manual_seed(123)
    q_idx = torch.randint(-3, 4, (1, n_tokens, 2, 8), generator=g).float()
    k_idx = torch.randint(-3, 4, (1, n_tokens, 2, 8), generator=g).float()
    w = torch.randint(0, 9, (1, n_tokens, 2), generator=g).float() / 8
    q, k, v = [torch.randn(1, n_tokens, 2, 8, generator=g) for _ in range(3)]
    idx_ref, _ = orc.indexer_topk(q_idx, k_idx, w, 5, 0.5)
    out_ref, _, _ = orc.sparse_attention(q, k, v, idx_ref, 0.5)
    out = torch.cat([res[r][0] for r in range(world)], 1)
    idx = torch.cat([res[r][1] for r in range(world)], 1)
    assert torch.equal(idx, idx_ref)
    torch.testing.assert_close(out, out_ref)


def test_wrong_shard_size_is_refused_before_communicating():
    res = _run(2, 10, "bad_shard")
    assert list(res.values())[0].startswith("raised")
