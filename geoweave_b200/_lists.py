"""Index lists grouped by key: the fixed order in which the backward kernels sum over the queries that selected a key."""
from __future__ import annotations

from typing import Tuple

import torch

from . import _lib


def group_by_key(positions: torch.Tensor, n_keys: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """positions: int32 ``[B,T,K]`` on the device (entries < 0 or >= n_keys are padding).  Returns ``(order, start)``:
    ``order`` int32 ``[B,T*K]``, the flat positions ``t*K + j`` stably sorted by key with padding entries last, and
    ``start`` int32 ``[B,n_keys+1]``, the first entry of every key in ``order`` (``start[:, n_keys]`` is where the padding
    begins).  The sort is stable, so the pairs of a key stay in (query, slot) order and sums taken in this order are
    reproducible.  One library call (``gw_group_by_key``: a radix sort over the bits a key can have, then the offsets)."""
    dev = _lib.require_cuda(positions)
    B, T, K = positions.shape
    lib = _lib.load()
    positions = positions.to(torch.int32).contiguous()
    order = torch.empty((B, T * K), device=dev, dtype=torch.int32)
    start = torch.empty((B, n_keys + 1), device=dev, dtype=torch.int32)
    ws = torch.empty(max(int(lib.gw_group_by_key_workspace_bytes(T, K, n_keys)), 1), device=dev, dtype=torch.uint8)
    with torch.cuda.device(dev):
        rc = lib.gw_group_by_key(positions.data_ptr(), B, T, K, n_keys, order.data_ptr(), start.data_ptr(), ws.data_ptr(),
                                 ws.numel(), _lib.stream_ptr(dev))
    _lib.check(rc, "gw_group_by_key")
    return order, start
