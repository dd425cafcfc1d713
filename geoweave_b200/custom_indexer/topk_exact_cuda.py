"""Exact top-k of a materialised score tensor -- same interface as the reference module
``easyvolcap/utils/custom_indexer/topk_exact_cuda.py`` (:48-85), without its k = 512 restriction.

K is taken from ``out_pos`` / ``out_scores`` when given, otherwise it is 512 (the reference's fixed size),
clipped to the row length.  Ties keep the lower column.  The order inside a row is unspecified.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _lib

_EXT_LOAD_ERROR = None
DEFAULT_K = 512


def _load_extension():
    global _EXT_LOAD_ERROR
    try:
        return _lib.load()
    except Exception as exc:
        _EXT_LOAD_ERROR = exc
        return None


def is_topk_exact_available() -> bool:
    return _load_extension() is not None


def topk_exact_select(scores: torch.Tensor, out_scores: Optional[torch.Tensor] = None,
                      out_pos: Optional[torch.Tensor] = None, k: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """scores ``[B,T,C]`` -> ``(out_scores [B,T,K] of scores.dtype, out_pos [B,T,K] int64 or int32)``."""
    lib = _load_extension()
    if lib is None:
        raise RuntimeError(f"topk_exact extension unavailable: {_EXT_LOAD_ERROR!r}")
    if scores.ndim != 3:
        raise ValueError(f"scores must be 3D, got shape={tuple(scores.shape)}")
    if not scores.is_cuda:
        raise ValueError("scores must be CUDA tensor")
    if not scores.is_contiguous():
        scores = scores.contiguous()
    bsz, rows, cols = scores.shape
    if k is None:
        k = out_pos.shape[-1] if out_pos is not None else (out_scores.shape[-1] if out_scores is not None else DEFAULT_K)
    k = int(k)
    if cols < k:
        raise ValueError(f"scores last dim must be >= {k}, got {cols}")
    if out_scores is None:
        out_scores = torch.empty((bsz, rows, k), device=scores.device, dtype=scores.dtype)
    if out_pos is None:
        out_pos = torch.empty((bsz, rows, k), device=scores.device, dtype=torch.long)
    for name, t in (("out_scores", out_scores), ("out_pos", out_pos)):
        if tuple(t.shape) != (bsz, rows, k) or not t.is_contiguous():
            raise ValueError(f"{name} must be a contiguous [B,T,{k}] tensor")
    if out_scores.dtype != scores.dtype:
        raise TypeError("out_scores dtype must match scores")
    if out_pos.dtype not in (torch.int64, torch.int32):
        raise TypeError("out_pos must be int64 or int32")
    p32 = out_pos.data_ptr() if out_pos.dtype == torch.int32 else None
    p64 = out_pos.data_ptr() if out_pos.dtype == torch.int64 else None
    with torch.cuda.device(scores.device):
        rc = lib.gw_topk_exact(scores.data_ptr(), _lib.dtype_code(scores), bsz * rows, cols, cols, k, p32, p64,
                               out_scores.data_ptr(), _lib.stream_ptr(scores.device))
    _lib.check(rc, "gw_topk_exact")
    return out_scores, out_pos
