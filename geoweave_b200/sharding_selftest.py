"""Self-test of the peer-memory exchange on the GPUs of one node:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m geoweave_b200.sharding_selftest [--iters 2000]

Every iteration draws new shard contents (and, every so often, a new shard size), exchanges them with ``PeerExchange``
-- the K_idx / w pair through the pull kernel, the K / V pair through copy engines, started asynchronously and joined
later, as the sharded layer does -- and compares with what NCCL's all-gather returns.  Rank 0 prints one line.
"""
from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=2000)
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    import geoweave_b200
    from geoweave_b200.sharding import PeerExchange, gather_rows, row_partition

    ex_idx, ex_kv = PeerExchange(device=dev, pull="kernel"), PeerExchange(device=dev, pull="copies", copy_streams=4)
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    host = torch.Generator().manual_seed(99)  # the same on every rank: the sizes
    n_rows = 1041 * world + 3                  # ragged: the first three ranks hold one row more
    bad = 0
    for it in range(args.iters):
        if it % 97 == 0:
            n_rows = int(torch.randint(world, 6000 * world, (1,), generator=host).item())
        lo, hi = row_partition(n_rows, world)[rank]
        rows = hi - lo
        k_idx = torch.randn(1, rows, 4, 64, device=dev, generator=gen).bfloat16()
        w = torch.randn(1, rows, 4, device=dev, generator=gen).bfloat16()
        k = torch.randn(1, rows, 16, 64, device=dev, generator=gen).bfloat16()
        v = torch.randn(1, rows, 16, 64, device=dev, generator=gen).bfloat16()
        got_i = ex_idx.gather([k_idx, w], n_rows).result()
        pend = ex_kv.gather([k, v], n_rows, async_op=True)
        want = [gather_rows(x, n_rows) for x in (k_idx, w, k, v)]   # NCCL, while the copies run
        got = got_i + pend.result()
        if not all(torch.equal(a, b) for a, b in zip(got, want)):
            bad += 1
    torch.cuda.synchronize()
    geoweave_b200.check_status()
    total = torch.tensor([bad], device=dev)
    dist.all_reduce(total)
    if rank == 0:
        print(f"peer exchange self-test: {args.iters} iterations on {world} GPUs, {int(total.item())} mismatches", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    if int(total.item()):
        raise SystemExit(1)


if __name__ == "__main__":
    main()
