"""Merge a running top-k list with a pending one -- same interface as the reference module
``easyvolcap/utils/custom_indexer/merge_two_topk_cuda.py`` (:48-83), for any k.

Like the reference, the function reports failure by returning ``False`` instead of raising.
"""
from __future__ import annotations

import os

import torch

from .. import _lib

_EXT_LOAD_ERROR = None
_EXT_CALL_ERROR_COUNT = 0


def _load_extension():
    global _EXT_LOAD_ERROR
    try:
        return _lib.load()
    except Exception as exc:
        _EXT_LOAD_ERROR = exc
        return None


def is_merge_two_topk_available() -> bool:
    return _load_extension() is not None


def merge_two_topk_inplace(topk_scores: torch.Tensor, topk_indices: torch.Tensor, pending_scores: torch.Tensor,
                           pending_pos: torch.Tensor, pending_start: int, out_scores: torch.Tensor,
                           out_indices: torch.Tensor) -> bool:
    """Keep the best K of ``topk ∪ (pending_pos + pending_start)``; all tensors ``[B,T,K*]`` contiguous,
    ``topk_indices``/``out_indices`` int32, ``pending_pos`` int64.  Outputs may alias the running list."""
    global _EXT_CALL_ERROR_COUNT
    lib = _load_extension()
    if lib is None:
        if os.getenv("VGGT_INDEXER_MERGE_TWO_DEBUG", "0") == "1":
            print("[merge_two_topk_cuda] extension unavailable:", repr(_EXT_LOAD_ERROR))
        return False
    try:
        tensors = (topk_scores, topk_indices, pending_scores, pending_pos, out_scores, out_indices)
        if not all(t.is_cuda and t.dim() == 3 and t.is_contiguous() for t in tensors):
            raise ValueError("all arguments must be contiguous 3-D CUDA tensors")
        if topk_indices.dtype != torch.int32 or out_indices.dtype != torch.int32 or pending_pos.dtype != torch.int64:
            raise TypeError("topk_indices/out_indices must be int32 and pending_pos int64")
        if not (topk_scores.dtype == pending_scores.dtype == out_scores.dtype):
            raise TypeError("scores dtype mismatch")
        b, t, ka = topk_scores.shape
        kb = pending_scores.shape[-1]
        k = out_scores.shape[-1]
        if topk_indices.shape != topk_scores.shape or pending_pos.shape != pending_scores.shape \
                or out_indices.shape != out_scores.shape or pending_scores.shape[:2] != (b, t) or out_scores.shape[:2] != (b, t):
            raise ValueError("shape mismatch")
        with torch.cuda.device(topk_scores.device):
            rc = lib.gw_merge_two_topk(topk_scores.data_ptr(), topk_indices.data_ptr(), ka, pending_scores.data_ptr(),
                                       pending_pos.data_ptr(), kb, int(pending_start), _lib.dtype_code(topk_scores), b * t,
                                       k, out_scores.data_ptr(), out_indices.data_ptr(),
                                       _lib.stream_ptr(topk_scores.device))
        _lib.check(rc, "gw_merge_two_topk")
        return True
    except Exception as exc:
        _EXT_CALL_ERROR_COUNT += 1
        if os.getenv("VGGT_INDEXER_MERGE_TWO_DEBUG", "0") == "1" and _EXT_CALL_ERROR_COUNT <= 8:
            print("[merge_two_topk_cuda] call failed:", repr(exc))
        return False
