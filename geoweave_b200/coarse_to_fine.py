"""Coarse-to-fine selection: rank 2x2-pooled patch cells with the indexer, then expand the kept cells to tokens.

The reference runs this reduction of stage 1 in its caller for long contexts (``source_downsample_enabled``, factor 2,
strategy ``legacy``; ``easyvolcap/official_vggt/layers/dsa_attention.py:3044-3258, 3328-3543, 4079-4128, 4187-4224``):
the coarse stage scores every query against ``L ~ N / 3.8`` "sources" instead of N keys -- every special token and every
patch token outside the pooled region as they are, every 2x2 cell of patches as the mean of its four tokens' indexer
keys and weights -- keeps ``ceil(topk / avg_expand * 1.1)`` of them and expands those round-robin (first token of every
kept source, then the second of every kept cell, ...) to exactly ``topk`` token indices.

Here: the source table is built once per token layout, the pooled keys come from one kernel (``gw_pool_sources``), the
coarse stage is the fused indexer kernel itself on ``[N queries] x [L sources]``, and the expansion is one kernel
(``gw_expand_sources``).  One deliberate difference: the reference expands the kept sources in whatever order its
unsorted top-k returned them, so which tokens survive the cut to ``topk`` is unspecified there; here the kept sources
are ordered by descending coarse score (equal scores: lower source index first), which makes the result deterministic
and drops the weakest sources' later tokens first.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from . import _lib
from .custom_indexer.sparse_topk_indexer import fused_score_topk

__all__ = ["SourceLayout", "source_layout", "pool_sources", "expand_sources", "select_topk_coarse_to_fine"]


@dataclass(frozen=True)
class SourceLayout:
    """Which tokens each source of the coarse stage stands for (``_get_source_downsample_layout``, :3069-3258)."""
    tokens_per_view: int
    num_views: int
    patch_start: int          # special tokens in front of every view's patches
    grid_h: int
    grid_w: int
    special_count: int
    edge_count: int           # patch tokens outside the pooled region (an odd last row / column)
    coarse_count: int         # 2x2 cells
    table: torch.Tensor       # int32 [source_len, 4] on the device: tokens of every source, -1 = no such slot
    token_source: torch.Tensor  # int64 [n_tokens] on the device: the source every token belongs to

    @property
    def source_len(self) -> int:
        return self.special_count + self.edge_count + self.coarse_count

    @property
    def n_tokens(self) -> int:
        return self.tokens_per_view * self.num_views

    @property
    def avg_expand(self) -> float:
        return (self.special_count + self.edge_count + 4 * self.coarse_count) / self.source_len

    def kept_sources(self, topk: int, ratio: float = 1.1) -> int:
        """How many sources the coarse stage keeps for ``topk`` tokens (``_resolve_source_downsample_coarse_topk``,
        :3328-3375, automatic budget)."""
        m = int(math.ceil(topk / max(self.avg_expand, 1.0) * max(ratio, 1.0)))
        special = min(self.special_count, topk)
        others = self.source_len - self.special_count
        if 0 < special < topk and m < special and others > 0:
            per_source = max((self.edge_count + 4 * self.coarse_count) / others, 1.0)
            m = max(m, special + max(int(math.ceil((topk - special) / per_source * max(ratio, 1.0))), 1))
        return min(max(m, 1), self.source_len)


_LAYOUTS: Dict[Tuple, SourceLayout] = {}


def source_layout(tokens_per_view: int, num_views: int, patch_start: int, grid_h: int, grid_w: int, device) -> SourceLayout:
    """Sources in the reference's order: all views' special tokens, then all views' patch tokens outside the pooled
    region (row-major), then all views' 2x2 cells (row-major), each cell's tokens row-major.  Cached per layout and device."""
    device = torch.device(device)
    key = (tokens_per_view, num_views, patch_start, grid_h, grid_w, device.type, device.index)
    hit = _LAYOUTS.get(key)
    if hit is not None:
        return hit
    if patch_start < 0 or grid_h <= 0 or grid_w <= 0 or tokens_per_view - patch_start != grid_h * grid_w or num_views <= 0:
        raise ValueError(f"tokens_per_view={tokens_per_view} is not {patch_start} special tokens + a {grid_h}x{grid_w} patch grid")
    ph, pw = grid_h // 2 * 2, grid_w // 2 * 2
    view0 = torch.arange(num_views, dtype=torch.int64).view(-1, 1) * tokens_per_view
    special = (view0 + torch.arange(patch_start).view(1, -1)).reshape(-1)
    ys, xs = torch.meshgrid(torch.arange(grid_h), torch.arange(grid_w), indexing="ij")
    outside = (ys >= ph) | (xs >= pw)
    edge = (view0 + patch_start + (ys * grid_w + xs)[outside].view(1, -1)).reshape(-1)
    cy, cx = torch.meshgrid(torch.arange(ph // 2), torch.arange(pw // 2), indexing="ij")
    corner = (2 * cy * grid_w + 2 * cx).reshape(1, -1, 1)
    cells = (view0.view(-1, 1, 1) + patch_start + corner + torch.tensor([0, 1, grid_w, grid_w + 1]).view(1, 1, 4)).reshape(-1, 4)
    table = torch.full((special.numel() + edge.numel() + cells.shape[0], 4), -1, dtype=torch.int64)
    table[: special.numel(), 0] = special
    table[special.numel(): special.numel() + edge.numel(), 0] = edge
    table[special.numel() + edge.numel():] = cells
    token_source = torch.empty(tokens_per_view * num_views, dtype=torch.int64)
    rows = torch.arange(table.shape[0]).view(-1, 1).expand_as(table)
    token_source[table[table >= 0]] = rows[table >= 0]
    lay = SourceLayout(tokens_per_view, num_views, patch_start, grid_h, grid_w, int(special.numel()), int(edge.numel()),
                       int(cells.shape[0]), table.to(torch.int32).to(device).contiguous(), token_source.to(device))
    _LAYOUTS[key] = lay
    return lay


def pool_sources(k_idx: torch.Tensor, w: Optional[torch.Tensor], layout: SourceLayout) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """``k_idx [B,N,Hi,Di]``, ``w [B,N,Hi]`` -> the sources' keys ``[B,L,Hi,Di]`` and weights ``[B,L,Hi]``
    (``_prepare_source_downsample_projected``, :3386-3543).  With ``w`` None only the first is made -- the same mean
    applied to the queries (``_prepare_query_downsample_chunk``, :3925-3994, for a chunk that holds whole sources)."""
    dev = _lib.require_cuda(k_idx) if w is None else _lib.require_cuda(k_idx, w)
    B, N, Hi, Di = k_idx.shape
    if N != layout.n_tokens or (w is not None and (tuple(w.shape) != (B, N, Hi) or w.dtype != k_idx.dtype)):
        raise ValueError(f"k_idx {tuple(k_idx.shape)} / w do not match a layout of {layout.n_tokens} tokens")
    if layout.table.device != dev:
        raise ValueError("the layout was built for another device")
    k_idx = k_idx.contiguous()
    w = None if w is None else w.contiguous()
    L = layout.source_len
    src_k = torch.empty((B, L, Hi, Di), device=dev, dtype=k_idx.dtype)
    src_w = None if w is None else torch.empty((B, L, Hi), device=dev, dtype=w.dtype)
    with torch.cuda.device(dev):
        rc = _lib.load().gw_pool_sources(k_idx.data_ptr(), _lib.ptr(w), layout.table.data_ptr(), _lib.dtype_code(k_idx), B, N, L, Hi,
                                         Di, 4, src_k.data_ptr(), _lib.ptr(src_w), _lib.stream_ptr(dev))
    _lib.check(rc, "gw_pool_sources")
    return src_k, src_w


def expand_sources(kept: torch.Tensor, scores: Optional[torch.Tensor], layout: SourceLayout, topk: int,
                   pad_window: int = 64) -> torch.Tensor:
    """``kept`` int32 ``[B,T,m]`` sources per query (and their scores, or None to keep the given order) -> int32
    ``[B,T,min(topk,N)]`` token indices (``_expand_source_downsample_chunk``, :4079-4128, round-robin form)."""
    dev = _lib.require_cuda(kept)
    if kept.dtype != torch.int32 or kept.dim() != 3:
        raise TypeError("kept must be int32 [B,T,m]")
    B, T, m = kept.shape
    if scores is not None and (tuple(scores.shape) != (B, T, m) or scores.dtype not in (torch.float32, torch.bfloat16, torch.float16)):
        raise ValueError("scores must match kept and be float32, bfloat16 or float16")
    out_k = min(int(topk), layout.n_tokens)
    out = torch.empty((B, T, out_k), device=dev, dtype=torch.int32)
    if B * T == 0:
        return out
    kept = kept.contiguous()
    scores = None if scores is None else scores.contiguous()
    with torch.cuda.device(dev):
        rc = _lib.load().gw_expand_sources(kept.data_ptr(), _lib.ptr(scores), 0 if scores is None else _lib.dtype_code(scores),
                                           layout.table.data_ptr(), 4, layout.source_len, layout.n_tokens, B * T, m, out_k,
                                           max(1, min(int(pad_window), out_k)), out.data_ptr(), _lib.stream_ptr(dev))
    _lib.check(rc, "gw_expand_sources")
    return out


def select_topk_coarse_to_fine(q_idx: torch.Tensor, k_idx: torch.Tensor, w: torch.Tensor, layout: SourceLayout, topk: int,
                               softmax_scale: Optional[float] = None, ratio: float = 1.1, pad_window: int = 64,
                               workspace: Optional[torch.Tensor] = None, pool_queries: bool = False) -> torch.Tensor:
    """The selection of a layer with pooled sources: int32 ``[B,T,min(topk,N)]`` token indices per query
    (``_select_topk_source_downsample_chunk``, :4187-4224).  ``k_idx`` / ``w`` are all N tokens of the layout.

    ``pool_queries=False`` (strategy ``legacy``): ``q_idx [B,T,Hi,Di]`` may be any block of query rows, each scored
    against the sources.  ``pool_queries=True`` (strategy ``qk_sym_x2_broadcast``, :4019-4077): the queries are pooled like
    the keys, one list is selected per source and every token takes the list of its source; ``q_idx`` must then be all N
    tokens."""
    src_k, src_w = pool_sources(k_idx, w, layout)
    m = layout.kept_sources(min(int(topk), layout.n_tokens), ratio)
    if not pool_queries:
        kept, scores = fused_score_topk(q_idx, src_k, src_w, m, softmax_scale, return_scores=True, workspace=workspace)
        return expand_sources(kept, scores, layout, topk, pad_window)
    src_q, _ = pool_sources(q_idx, None, layout)
    kept, scores = fused_score_topk(src_q, src_k, src_w, m, softmax_scale, return_scores=True, workspace=workspace)
    lists = expand_sources(kept, scores, layout, topk, pad_window)          # [B,L,topk]
    return lists.index_select(1, layout.token_source)                       # (:3996-4017)
