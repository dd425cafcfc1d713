"""Indexer score + exact top-k -- same call signatures as the reference module
``easyvolcap/utils/custom_indexer/sparse_topk_indexer.py`` (``sparse_topk_indexer_func`` :2188-2253) and the
inference slot ``sparse_topk_indexer_inference_func`` the reference leaves open
(``easyvolcap/utils/custom_indexer/__init__.py:4-7``, called at ``official_vggt/layers/indexer.py:570-581``).

One fused tcgen05 kernel computes ``score[t,s] = sum_h w[s,h] * relu(scale * q[t,h].k[s,h])`` tile by tile and
keeps the exact top-k per query in its epilogue; the score matrix is never written to memory.  The
``block_k`` / ``merge_blocks`` / ``outer_query_chunk`` arguments tune the reference's block-wise loop and have no
meaning here; they are accepted and ignored.  fp32 operands (the reference's torch backend) take a plain fp32 score
kernel followed by the exact top-k kernel instead.  ``mask`` and ``view_bias_data`` are not implemented (both
published presets run without them) and raise ``NotImplementedError`` -- there is no fallback path.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from .. import _lib
from .._lists import group_by_key

__all__ = ["sparse_topk_indexer_func", "sparse_topk_indexer_inference_func", "indexer_scores", "indexer_workspace_bytes",
           "indexer_topk_backward", "clear_runtime_cache"]

clear_runtime_cache = _lib.clear_runtime_cache


def _check_qkw(q, k, w):
    if q.dim() != 4 or k.dim() != 4 or w.dim() != 3:
        raise ValueError(f"invalid shapes q={tuple(q.shape)} k={tuple(k.shape)} w={tuple(w.shape)}; "
                         "expect q/k as [B,T(orS),H,D] and w as [B,S,H]")
    bq, tq, hq, dq = q.shape
    bk, sk, hk, dk = k.shape
    bw, sw, hw = w.shape
    if bq != bk or bq != bw or hq != hk or hq != hw or dq != dk or sk != sw:
        raise ValueError("q/k/w shape mismatch")
    if not (q.dtype == k.dtype == w.dtype):
        raise TypeError("q/k/w must share one dtype")
    if q.dtype not in (torch.bfloat16, torch.float16, torch.float32):
        raise TypeError(f"the indexer takes bfloat16, float16 or float32 inputs, got {q.dtype} "
                        "(scores are always accumulated in fp32)")
    return bq, tq, sk, hq, dq


_F32_SCORE_BYTES = 1 << 30  # fp32 operands: scores are materialised for this many bytes of query rows at a time


def _score_topk_f32(q, k, w, topk, scale, idx, sc):
    """fp32 operands (the reference's torch backend forces ``score_dtype=float32``, ``geoweave/inference.py:56-58``):
    dense fp32 scores of a block of query rows from an FFMA kernel, then the exact top-k kernel on them, block after
    block.  Far slower than the 16-bit tensor-core path and meant for the reference's small fp32 configuration."""
    lib = _lib.load()
    dev = q.device
    B, T, Hi, Di = q.shape
    S = k.shape[1]
    if Di != 64:
        raise _lib.GeoWeaveError(-2, "the indexer kernels are built for head_dim 64")
    chunk = max(64, min(T, _F32_SCORE_BYTES // (4 * S * B)) // 64 * 64)
    scratch = torch.empty(B * chunk * S, device=dev, dtype=torch.float32)
    stream = _lib.stream_ptr(dev)
    with torch.cuda.device(dev):
        for r0 in range(0, T, chunk):
            rows = min(chunk, T - r0)
            _lib.check(lib.gw_indexer_scores_f32(q.data_ptr(), k.data_ptr(), w.data_ptr(), B, T, S, Hi, Di, scale, r0, rows,
                                                 scratch.data_ptr(), S, stream), "gw_indexer_scores_f32")
            for b in range(B):
                rows_ptr = scratch.data_ptr() + 4 * b * rows * S
                _lib.check(lib.gw_topk_exact(rows_ptr, _lib.GW_F32, rows, S, S, topk, idx[b, r0:r0 + rows].data_ptr(), None,
                                             None if sc is None else sc[b, r0:r0 + rows].data_ptr(), stream), "gw_topk_exact")
    return idx, sc


def indexer_workspace_bytes(B: int, T: int, S: int, Hi: int, Di: int, topk: int) -> int:
    """Bytes of device workspace one ``fused_score_topk`` call of this shape needs."""
    return int(_lib.load().gw_indexer_topk_workspace_bytes(B, T, S, Hi, Di, min(int(topk), S)))


def fused_score_topk(q, k, w, topk: int, softmax_scale: Optional[float], return_scores: bool = True,
                     out_indices: Optional[torch.Tensor] = None, out_scores: Optional[torch.Tensor] = None,
                     workspace: Optional[torch.Tensor] = None):
    """q ``[B,T,Hi,Di]``, k ``[B,S,Hi,Di]``, w ``[B,S,Hi]`` -> (int32 ``[B,T,k]``, scores of q.dtype or None).

    ``workspace``: a uint8 tensor of at least ``indexer_workspace_bytes(...)`` that the caller owns (a captured CUDA
    graph keeps its own, so that nothing can replace it between replays); by default a buffer cached per
    (device, stream) is used.  Calls that may overlap on the GPU need different workspaces."""
    dev = _lib.require_cuda(q, k, w)
    B, T, S, Hi, Di = _check_qkw(q, k, w)
    q, k, w = q.contiguous(), k.contiguous(), w.contiguous()
    topk = min(int(topk), S)
    if topk <= 0:
        raise ValueError("topk must be positive")
    scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(Di)
    idx = out_indices if out_indices is not None else torch.empty((B, T, topk), device=dev, dtype=torch.int32)
    sc = out_scores if out_scores is not None else (
        torch.empty((B, T, topk), device=dev, dtype=q.dtype) if return_scores else None)
    if idx.dtype != torch.int32 or tuple(idx.shape) != (B, T, topk) or not idx.is_contiguous():
        raise ValueError(f"out_indices must be a contiguous int32 [B,T,{topk}] tensor")
    if sc is not None and (sc.dtype != q.dtype or tuple(sc.shape) != (B, T, topk) or not sc.is_contiguous()):
        raise ValueError(f"out_scores must be a contiguous {q.dtype} [B,T,{topk}] tensor")
    if T == 0:
        return idx, sc
    if q.dtype == torch.float32:
        return _score_topk_f32(q, k, w, topk, scale, idx, sc)
    lib = _lib.load()
    nbytes = int(lib.gw_indexer_topk_workspace_bytes(B, T, S, Hi, Di, topk))
    if workspace is None:
        ws = _lib.workspace(dev, nbytes)
    else:
        ws = workspace
        if ws.dtype != torch.uint8 or ws.device != dev or not ws.is_contiguous() or ws.numel() < nbytes:
            raise ValueError(f"workspace must be a contiguous uint8 tensor of at least {nbytes} bytes on {dev}")
    with torch.cuda.device(dev):
        rc = lib.gw_indexer_topk_fused(q.data_ptr(), k.data_ptr(), w.data_ptr(), _lib.dtype_code(q), B, T, S, Hi, Di,
                                       scale, topk, idx.data_ptr(), _lib.ptr(sc), ws.data_ptr(), ws.numel(),
                                       _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev))
    _lib.check(rc, "gw_indexer_topk_fused")
    if _lib.debug_enabled():
        _lib.check_status(dev)
    return idx, sc


def indexer_scores(q, k, w, softmax_scale: Optional[float] = None, key_step: int = 1) -> torch.Tensor:
    """Dense fp32 scores ``[B,T,ceil(S/key_step)]`` from the same tensor-core main loop (verification and
    threshold sampling; the counterpart of the reference's ``_compute_scores_block_einsum``, :935-951)."""
    dev = _lib.require_cuda(q, k, w)
    B, T, S, Hi, Di = _check_qkw(q, k, w)
    q, k, w = q.contiguous(), k.contiguous(), w.contiguous()
    scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(Di)
    m = (S + key_step - 1) // key_step
    out = torch.empty((B, T, m), device=dev, dtype=torch.float32)
    lib = _lib.load()
    if q.dtype == torch.float32:
        if key_step != 1:
            raise ValueError("key_step applies to the 16-bit tensor-core path only")
        with torch.cuda.device(dev):
            _lib.check(lib.gw_indexer_scores_f32(q.data_ptr(), k.data_ptr(), w.data_ptr(), B, T, S, Hi, Di, scale, 0, T,
                                                 out.data_ptr(), S, _lib.stream_ptr(dev)), "gw_indexer_scores_f32")
        return out
    with torch.cuda.device(dev):
        rc = lib.gw_indexer_scores(q.data_ptr(), k.data_ptr(), w.data_ptr(), _lib.dtype_code(q), B, T, S, Hi, Di, scale,
                                   int(key_step), out.data_ptr(), m, _lib.status_word(dev).data_ptr(),
                                   _lib.stream_ptr(dev))
    _lib.check(rc, "gw_indexer_scores")
    if _lib.debug_enabled():
        _lib.check_status(dev)
    return out


def _reject_mask(mask, view_bias_data):
    if mask is not None and mask.numel() != 0:
        raise NotImplementedError("an additive score mask is not implemented (presets run with sparse_use_mask=false)")
    if view_bias_data is not None:
        raise NotImplementedError("soft view bias is a training-time option and is not implemented")


def indexer_topk_backward(q, k, w, topk_indices, grad_scores, softmax_scale: Optional[float]):
    """Gradients of the selected scores ``score[t,j] = sum_h w[idx[t,j],h] * relu(scale * q[t,h].k[idx[t,j],h])`` with
    respect to q, k and w, given ``grad_scores`` ``[B,T,k]`` -- the reference's ``_backward_selected_topk_qkw`` (:757-895).
    Entries of ``topk_indices`` outside ``[0, S)`` carry no gradient.  The sums over the queries that selected a key run
    in a fixed order (no floating-point atomics), so the result is reproducible.  16-bit operands, head_dim 64, at most
    four heads."""
    dev = _lib.require_cuda(q, k, w, topk_indices, grad_scores)
    B, T, S, Hi, Di = _check_qkw(q, k, w)
    if q.dtype == torch.float32 or Di != 64 or Hi > 4:
        raise NotImplementedError("the indexer's backward kernels take bfloat16 / float16 operands with head_dim 64 and "
                                  "at most 4 heads")
    if topk_indices.dtype != torch.int32 or topk_indices.dim() != 3 or topk_indices.shape[:2] != (B, T):
        raise ValueError("topk_indices must be int32 [B,T,k]")
    K = topk_indices.shape[-1]
    if tuple(grad_scores.shape) != (B, T, K):
        raise ValueError(f"grad_scores must be [B,T,{K}], got {tuple(grad_scores.shape)}")
    q, k, w, topk_indices = q.contiguous(), k.contiguous(), w.contiguous(), topk_indices.contiguous()
    g = grad_scores.to(torch.float32).contiguous()
    dq, dk, dw = torch.empty_like(q), torch.empty_like(k), torch.empty_like(w)
    if T == 0 or K == 0:
        return dq.zero_(), dk.zero_(), dw.zero_()
    order, start = group_by_key(topk_indices, S)
    scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(Di)
    lib = _lib.load()
    ws = torch.empty(int(lib.gw_indexer_topk_bwd_workspace_bytes(B, T, S, K)), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        rc = lib.gw_indexer_topk_bwd(q.data_ptr(), k.data_ptr(), w.data_ptr(), topk_indices.data_ptr(), g.data_ptr(),
                                     order.data_ptr(), start.data_ptr(), _lib.dtype_code(q), B, T, S, Hi, Di, K, scale,
                                     dq.data_ptr(), dk.data_ptr(), dw.data_ptr(), ws.data_ptr(), ws.numel(),
                                     _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev))
    _lib.check(rc, "gw_indexer_topk_bwd")
    if _lib.debug_enabled():
        _lib.check_status(dev)
    return dq, dk, dw


class _SparseTopkIndexer(torch.autograd.Function):
    """The reference's ``SparseTopkIndexerFunc`` (:2047-2106): the selection itself runs without a graph, the returned
    scores are differentiable in q, k and w."""

    @staticmethod
    def forward(ctx, q, k, w, topk, softmax_scale):
        q, k, w = q.contiguous(), k.contiguous(), w.contiguous()
        idx, sc = fused_score_topk(q, k, w, topk, softmax_scale, return_scores=True)
        ctx.save_for_backward(q, k, w, idx)
        ctx.softmax_scale = softmax_scale
        ctx.mark_non_differentiable(idx)
        ctx.set_materialize_grads(False)
        return idx, sc

    @staticmethod
    def backward(ctx, grad_indices, grad_scores):
        if grad_scores is None:
            return None, None, None, None, None
        q, k, w, idx = ctx.saved_tensors
        dq, dk, dw = indexer_topk_backward(q, k, w, idx, grad_scores, ctx.softmax_scale)
        return dq, dk, dw, None, None


def sparse_topk_indexer_func(q: torch.Tensor, k: torch.Tensor, w: torch.Tensor, mask: Optional[torch.Tensor], topk: int,
                             softmax_scale: Optional[float], block_k: int, merge_blocks: int = 0,
                             view_bias_data: Optional[dict] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(topk_indices int32 [B,T,k], topk_scores q.dtype [B,T,k])``.  With inputs that require grad the scores
    are differentiable in q, k and w (16-bit operands); the selection itself is computed without a graph, as in the
    reference (:2071)."""
    _reject_mask(mask, view_bias_data)
    if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or w.requires_grad):
        if q.dtype == torch.float32:
            raise NotImplementedError("the indexer's backward kernels take bfloat16 / float16 operands")
        return _SparseTopkIndexer.apply(q, k, w, topk, softmax_scale)
    with torch.no_grad():
        return fused_score_topk(q, k, w, topk, softmax_scale, return_scores=True)


@torch.inference_mode()
def sparse_topk_indexer_inference_func(q, k, w, mask, topk, softmax_scale, topk_block=0, topk_merge_blocks=0,
                                       outer_query_chunk: int = 0, return_scores: bool = True):
    """Inference entry: ``(indices, scores | None)``."""
    _reject_mask(mask, None)
    return fused_score_topk(q, k, w, topk, softmax_scale, return_scores=return_scores)
