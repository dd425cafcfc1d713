"""Index lists grouped by key: the fixed order in which the backward kernels sum over the queries that selected a key."""
from __future__ import annotations

from typing import Tuple

import torch


def group_by_key(positions: torch.Tensor, n_keys: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """positions: int32 ``[B,T,K]`` (entries < 0 or >= n_keys are padding).  Returns ``(order, start)``: ``order`` int32
    ``[B,T*K]``, the flat positions ``t*K + j`` stably sorted by key with padding entries last, and ``start`` int32
    ``[B,n_keys+1]``, the first entry of every key in ``order`` (``start[:, n_keys]`` is where the padding begins).
    The sort is stable, so the pairs of a key stay in (query, slot) order and sums taken in this order are reproducible."""
    B, T, K = positions.shape
    dev = positions.device
    if positions.is_cuda:
        from . import _lib

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
    # host tensors (the CPU tests of the bookkeeping): the same result from torch's stable sort
    flat = positions.reshape(B, T * K).to(torch.int32)  # 32-bit keys: half the passes of the radix sort
    flat = torch.where((flat < 0) | (flat >= n_keys), torch.full_like(flat, n_keys), flat)
    keys_sorted, order = torch.sort(flat, dim=1, stable=True)
    bounds = torch.arange(n_keys + 1, device=dev, dtype=torch.int32).unsqueeze(0).expand(B, n_keys + 1).contiguous()
    start = torch.searchsorted(keys_sorted, bounds, out_int32=True).contiguous()
    return order.to(torch.int32).contiguous(), start
