"""Multi-GPU form of the path: query rows are split into contiguous slices, one per rank; every rank needs
all keys, so K_idx with w, and K with V, are all-gathered once per layer and nothing else is exchanged -- either as two
NCCL collectives or, on one node, pulled from peer memory behind a flag barrier (``PeerExchange``).  The reference has no multi-GPU form of this op; the split follows its own single-GPU
query-chunk loop, which keeps K/V/K_idx resident and walks query chunks
(easyvolcap/official_vggt/layers/dsa_attention.py:1138-1264, ``_run_sparse_streaming_direct``).
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist

__all__ = ["row_partition", "shard_rows", "gather_rows", "gather_rows_async", "gather_rows_packed", "gather_rows_group",
           "PeerExchange", "sparse_global_attention_sharded"]


def row_partition(n_rows: int, world_size: int) -> List[Tuple[int, int]]:
    """Contiguous [start, stop) per rank; the first ``n_rows % world_size`` ranks get one extra row."""
    if n_rows < 0 or world_size <= 0:
        raise ValueError("n_rows must be >= 0 and world_size > 0")
    base, extra = divmod(n_rows, world_size)
    out, start = [], 0
    for r in range(world_size):
        size = base + (1 if r < extra else 0)
        out.append((start, start + size))
        start += size
    return out


def shard_rows(x: torch.Tensor, rank: int, world_size: int, dim: int = 1) -> torch.Tensor:
    lo, hi = row_partition(x.shape[dim], world_size)[rank]
    return x.narrow(dim, lo, hi - lo)


class _PendingGather:
    """Handle of an all-gather in flight; ``result()`` waits for it and returns the full tensor."""

    def __init__(self, work, finish):
        self._work, self._finish, self._out = work, finish, None

    def result(self) -> torch.Tensor:
        if self._out is None:
            if self._work is not None:
                self._work.wait()
            self._out = self._finish()
        return self._out


def gather_rows_async(x: torch.Tensor, n_rows: int, group=None, dim: int = 1) -> _PendingGather:
    """``gather_rows`` that returns at once: the collective runs on the communication stream while the caller
    launches independent kernels (the indexer needs only K_idx and w; K and V can arrive behind it)."""
    return _gather_rows(x, n_rows, group, dim, True)


def gather_rows(x: torch.Tensor, n_rows: int, group=None, dim: int = 1) -> torch.Tensor:
    return _gather_rows(x, n_rows, group, dim, False).result()


def _gather_rows(x: torch.Tensor, n_rows: int, group, dim: int, async_op: bool) -> _PendingGather:
    """All-gather row shards (``row_partition`` sizes along ``dim``) into the full ``n_rows`` tensor.

    Equal shards go through one ``all_gather_into_tensor``; ragged shards are padded to the largest and
    trimmed afterwards.  Every rank must call this with the same ``n_rows``; a shard whose size disagrees
    with the partition raises before any communication.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    parts = row_partition(n_rows, world)
    lo, hi = parts[rank]
    if x.shape[dim] != hi - lo:
        raise ValueError(f"rank {rank}: shard has {x.shape[dim]} rows, partition of {n_rows} over {world} expects {hi - lo}")
    if world == 1:
        return _PendingGather(None, lambda: x)
    xm = x.movedim(dim, 0).contiguous()
    biggest = max(b - a for a, b in parts)
    if xm.shape[0] < biggest:
        pad = torch.zeros((biggest - xm.shape[0],) + tuple(xm.shape[1:]), dtype=xm.dtype, device=xm.device)
        xm = torch.cat([xm, pad], 0)
    out = torch.empty((world * biggest,) + tuple(xm.shape[1:]), dtype=xm.dtype, device=xm.device)
    if xm.is_cuda:
        work = dist.all_gather_into_tensor(out, xm, group=group, async_op=async_op)
    else:  # gloo (CPU tests)
        chunks = list(out.chunk(world, 0))
        work = dist.all_gather(chunks, xm, group=group, async_op=async_op)

    def finish():
        full = out
        if any(b - a != biggest for a, b in parts):
            full = torch.cat([out[r * biggest: r * biggest + (b - a)] for r, (a, b) in enumerate(parts)], 0)
        return full.movedim(0, dim)

    return _PendingGather(work if async_op else None, finish)


class _PendingPacked:
    def __init__(self, pending: _PendingGather, split):
        self._pending, self._split, self._out = pending, split, None

    def result(self):
        if self._out is None:
            self._out = self._split(self._pending.result())
        return self._out


def gather_rows_packed(xs: Sequence[torch.Tensor], n_rows: int, group=None, async_op: bool = False) -> _PendingPacked:
    """All-gather several row-sharded tensors ``[B, rows, ...]`` of one dtype with ONE collective: each token's values
    are laid side by side, gathered, and handed back as views of the gathered buffer (token stride = the packed
    width; the last dimension of every view stays contiguous, which is all the attention operator asks of K and V).
    One collective instead of two saves a launch and a latency per layer, which shows at eight ranks where the
    whole layer takes under 2 ms.  ``result()`` returns the list of full tensors."""
    xs = list(xs)
    if len({x.dtype for x in xs}) != 1 or len({tuple(x.shape[:2]) for x in xs}) != 1:
        raise ValueError("packed tensors must share dtype, batch and row count")
    B, rows = xs[0].shape[:2]
    widths = [int(x[0, 0].numel()) if rows > 0 else int(torch.Size(x.shape[2:]).numel()) for x in xs]
    tails = [tuple(x.shape[2:]) for x in xs]
    packed = torch.cat([x.reshape(B, rows, wd) for x, wd in zip(xs, widths)], dim=-1)
    pending = _gather_rows(packed, n_rows, group, 1, async_op)

    def split(full):
        out, off = [], 0
        for wd, tail in zip(widths, tails):
            out.append(full[:, :, off: off + wd].unflatten(-1, tail) if len(tail) != 1 else full[:, :, off: off + wd])
            off += wd
        return out

    return _PendingPacked(pending, split)


class _PendingGroup:
    def __init__(self, work, outs):
        self._work, self._outs = work, outs

    def result(self):
        if self._work is not None:
            self._work.wait()
            self._work = None
        return self._outs


def gather_rows_group(xs: Sequence[torch.Tensor], n_rows: int, group=None, async_op: bool = False):
    """All-gather several row-sharded tensors ``[B, rows, ...]`` as ONE exchange step whose results are separate,
    contiguous full tensors -- no packing copy in front and no un-packing copy behind.  With NCCL and equal shards the
    all-gathers are issued as one coalesced group (one launch); batches larger than 1, ragged shards and other
    back ends go through ``gather_rows_packed``.  ``result()`` returns the list of full tensors."""
    xs = list(xs)
    world = dist.get_world_size(group)
    B, rows = xs[0].shape[:2]
    equal = n_rows % world == 0 and rows * world == n_rows
    if world == 1 or B != 1 or not equal or not all(x.is_cuda and x.is_contiguous() for x in xs):
        if world > 1 and len({x.dtype for x in xs}) != 1:  # the packed form needs one dtype: gather one by one
            return _PendingGroup(None, [gather_rows(x, n_rows, group) for x in xs])
        return gather_rows_packed(xs, n_rows, group, async_op)
    if any(x.shape[1] != rows for x in xs):
        raise ValueError("gathered tensors must share the row count")
    outs = [torch.empty((1, n_rows) + tuple(x.shape[2:]), dtype=x.dtype, device=x.device) for x in xs]
    manager = getattr(dist, "_coalescing_manager", None)
    if manager is None:
        works = [dist.all_gather_into_tensor(o, x, group=group, async_op=async_op) for o, x in zip(outs, xs)]
        return _PendingGroup(works[-1] if async_op else None, outs)  # one communication stream: the last one finishes last
    with manager(group=group, async_ops=async_op) as cm:  # NCCL has a coalesced all-gather: one launch for the group
        for o, x in zip(outs, xs):
            dist.all_gather_into_tensor(o, x, group=group)
    return _PendingGroup(cm if async_op else None, outs)


class _PendingPeer:
    def __init__(self, exchange, outs, keep):
        self._exchange, self._outs, self._keep = exchange, outs, keep

    def result(self):
        if self._exchange is not None:
            self._exchange._join()
            self._exchange = self._keep = None
        return self._outs


class PeerExchange:
    """The layer's exchange step over peer memory instead of NCCL (GPUs of one node, one process per GPU).

    Every rank keeps its shard in a buffer that all ranks have mapped (``torch.distributed._symmetric_memory``: CUDA
    virtual-memory handles exchanged once, at construction).  ``gather`` then (1) copies the rank's rows into its own
    buffer, (2) meets the other ranks in a barrier kernel of this library that signals through flags in peer memory
    (bounded waits that report ``GW_ERR_TIMEOUT``), and (3) PULLS every peer's rows into the full tensors:

    * ``pull="copies"``: device-to-device copies spread over ``copy_streams`` streams, which the driver runs on copy
      engines over NVLink -- no SM is taken from the kernel that runs beside the exchange (K and V arrive while the
      indexer runs, and the indexer keeps its speed);
    * ``pull="kernel"``: one kernel that reads all peers -- for the small exchange in front of the indexer (K_idx, w),
      where nothing runs beside it and a 17 MB exchange should not pay a collective's protocol latency.

    Buffers alternate between two halves, so one barrier per exchange is enough: a rank overwrites a half only after the
    next exchange's barrier, which no peer passes before its reads of that half are done.  Each instance serialises its
    exchanges; every rank must call ``gather`` in the same order with the same shapes, and must call ``result()`` of one
    exchange before starting the next on the same instance.  Batch size 1.  The whole step is enqueued by two library
    calls (``gw_peer_exchange_run`` / ``_join``)."""

    def __init__(self, group=None, device=None, pull: str = "copies", copy_streams: int = 4, limit_ms: int = 2000):
        import ctypes

        import torch.distributed._symmetric_memory as symm

        from . import _lib

        if pull not in ("copies", "kernel"):
            raise ValueError(pull)
        self._symm, self._lib, self._ct = symm, _lib, ctypes
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.limit_ms, self.pull_kernel = int(limit_ms), int(pull == "kernel")
        self.capacity, self.seq = 0, 0
        self.halves, self.handles = [], []
        self._handle = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().gw_peer_exchange_create(1 if self.pull_kernel else int(copy_streams), ctypes.byref(self._handle)),
                       "gw_peer_exchange_create")
        self.flags = symm.empty(64, dtype=torch.int32, device=self.device)
        self.flags.zero_()
        self.flag_handle = symm.rendezvous(self.flags, self.group)
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)  # every rank's zeroed flags exist before anyone signals

    def __del__(self):
        try:
            if self._handle:
                self._lib.load().gw_peer_exchange_destroy(self._handle)
                self._handle = None
        except Exception:
            pass

    def _reserve(self, nbytes: int) -> None:
        """Collective: grows the two data buffers (all ranks ask for the same size at the same call)."""
        if nbytes <= self.capacity:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)  # nobody still reads the old buffers
        self.capacity = (nbytes + (1 << 20) - 1) >> 20 << 20
        self.halves = [self._symm.empty(self.capacity, dtype=torch.uint8, device=self.device) for _ in range(2)]
        self.handles = [self._symm.rendezvous(h, self.group) for h in self.halves]

    def _join(self):
        with torch.cuda.device(self.device):
            rc = self._lib.load().gw_peer_exchange_join(self._handle, self._lib.stream_ptr(self.device), self.pull_kernel)
        self._lib.check(rc, "gw_peer_exchange_join")

    def gather(self, xs: Sequence[torch.Tensor], n_rows: int, async_op: bool = False) -> _PendingPeer:
        """All-gather row shards ``[1, rows_of_this_rank, ...]`` (``row_partition`` sizes) into separate contiguous full
        tensors ``[1, n_rows, ...]``.  ``result()`` makes the current stream wait for the exchange and returns them."""
        ct = self._ct
        xs = [x.contiguous() for x in xs]
        parts = row_partition(n_rows, self.world)
        lo, hi = parts[self.rank]
        biggest = max(b - a for a, b in parts)
        if any(x.shape[0] != 1 or x.shape[1] != hi - lo or x.device != self.device for x in xs):
            raise ValueError(f"rank {self.rank}: shards must be [1, {hi - lo}, ...] on {self.device}")
        row_bytes = [x.element_size() * int(torch.Size(x.shape[2:]).numel()) for x in xs]
        offs, total = [], 0
        for rb in row_bytes:
            offs.append(total)
            total += (biggest * rb + 255) // 256 * 256
        self._reserve(total)
        outs = [torch.empty((1, n_rows) + tuple(x.shape[2:]), dtype=x.dtype, device=self.device) for x in xs]
        half = self.seq & 1
        self.seq += 1
        mine = self.halves[half].data_ptr()
        bases = list(self.handles[half].buffer_ptrs)
        pack_src = [x.data_ptr() for x in xs]
        pack_dst = [mine + off for off in offs]
        pack_n = [(hi - lo) * rb for rb in row_bytes]
        pull_src, pull_dst, pull_n = [], [], []
        for step in range(self.world):  # every rank starts with another peer
            r = (self.rank + step) % self.world
            a, b = parts[r]
            base = mine if r == self.rank else bases[r]
            for out, off, rb in zip(outs, offs, row_bytes):
                pull_src.append(base + off)
                pull_dst.append(out.data_ptr() + a * rb)
                pull_n.append((b - a) * rb)
        arr = lambda typ, vals: (typ * len(vals))(*vals)
        with torch.cuda.device(self.device):
            rc = self._lib.load().gw_peer_exchange_run(
                self._handle, self._lib.stream_ptr(self.device), self.flag_handle.buffer_ptrs_dev, self.rank, self.world, self.seq,
                self.limit_ms, self._lib.status_word(self.device).data_ptr(), len(xs), arr(ct.c_void_p, pack_src), arr(ct.c_void_p, pack_dst),
                arr(ct.c_size_t, pack_n), len(pull_n), arr(ct.c_void_p, pull_src), arr(ct.c_void_p, pull_dst), arr(ct.c_size_t, pull_n),
                self.pull_kernel)
        self._lib.check(rc, "gw_peer_exchange_run")
        pending = _PendingPeer(self, outs, xs)
        if not async_op:
            pending.result()
        return pending


def sparse_global_attention_sharded(q_idx, k_idx, w, q, k, v, topk: int, n_tokens: int, group=None,
                                    idx_scale=None, attn_scale=None, ops=None, exchange=None):
    """One layer of the path on this rank's token shard (all tensors ``[B, rows_of_this_rank, ...]``).

    Returns ``(out [B, rows, H, D], indices int32 [B, rows, k])`` for this rank's query rows; indices are
    global key indices.  ``ops`` = (indexer, attention) callables, by default this library's CUDA ops (the
    CPU tests pass stand-ins to exercise the bookkeeping without a GPU).  ``exchange`` = a pair of ``PeerExchange``
    objects (for K_idx with w, and for K with V) to pull the rows from peer memory instead of calling NCCL.
    """
    if ops is None:
        from .custom_flash_attn import sparse_index_flash_attn_inference_func
        from .custom_indexer import sparse_topk_indexer_inference_func

        def indexer(qi, ki, ww, kk, sc):
            return sparse_topk_indexer_inference_func(qi, ki, ww, None, kk, sc, 0, 0, return_scores=False)[0]

        def attention(qq, kk_, vv, pos, sc):
            return sparse_index_flash_attn_inference_func(qq, kk_, vv, pos, None, False, sc, False)[0]
    else:
        indexer, attention = ops
    if exchange is not None:
        k_idx_full, w_full = exchange[0].gather([k_idx, w], n_tokens).result()
        kv_pending = exchange[1].gather([k, v], n_tokens, async_op=True)
    else:
        k_idx_full, w_full = gather_rows_group([k_idx, w], n_tokens, group).result()
        kv_pending = gather_rows_group([k, v], n_tokens, group, async_op=True)  # K and V arrive while the indexer runs
    idx = indexer(q_idx, k_idx_full.contiguous(), w_full.contiguous(), topk, idx_scale)
    k_full, v_full = kv_pending.result()
    out = attention(q, k_full, v_full, idx, attn_scale)
    return out, idx
