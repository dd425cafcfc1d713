"""Fused score + top-k -- same interface as the reference module
``easyvolcap/utils/custom_indexer/score_topk_fused_cuda.py`` (:48-99), for any K (taken from the output
tensors when given, else 512 as in the reference)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _lib
from .sparse_topk_indexer import fused_score_topk

_EXT_LOAD_ERROR = None
_EXT_CALL_ERROR_COUNT = 0
DEFAULT_K = 512


def _load_extension():
    global _EXT_LOAD_ERROR
    try:
        return _lib.load()
    except Exception as exc:
        _EXT_LOAD_ERROR = exc
        return None


def is_score_topk_fused_available() -> bool:
    return _load_extension() is not None


def score_topk_fused_select(q: torch.Tensor, k: torch.Tensor, w: torch.Tensor, *, softmax_scale: float,
                            out_scores: Optional[torch.Tensor] = None,
                            out_pos: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    global _EXT_CALL_ERROR_COUNT
    if _load_extension() is None:
        raise RuntimeError(f"score_topk_fused extension unavailable: {_EXT_LOAD_ERROR!r}")
    if q.ndim != 4 or k.ndim != 4 or w.ndim != 3:
        raise ValueError(f"invalid shapes q={tuple(q.shape)} k={tuple(k.shape)} w={tuple(w.shape)}; "
                         "expect q/k as [B,T(orS),H,D] and w as [B,S,H]")
    if not (q.is_cuda and k.is_cuda and w.is_cuda):
        raise ValueError("q/k/w must be CUDA tensors")
    kk = out_pos.shape[-1] if out_pos is not None else (out_scores.shape[-1] if out_scores is not None else DEFAULT_K)
    try:
        idx, sc = fused_score_topk(q, k, w, kk, float(softmax_scale), True, out_indices=out_pos, out_scores=out_scores)
    except (ValueError, TypeError, NotImplementedError):
        raise
    except Exception as exc:
        _EXT_CALL_ERROR_COUNT += 1
        raise RuntimeError(f"score_topk_fused call failed ({_EXT_CALL_ERROR_COUNT}): {exc!r}") from exc
    return sc, idx
