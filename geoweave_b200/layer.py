"""One sparse global-attention layer as a single call: fused projection -> front-end kernel -> indexer (or the
indices of an earlier layer) -> sparse attention, optionally replayed from a CUDA graph.

This is the composition the reference's fastest configuration runs per layer
(``easyvolcap/official_vggt/layers/dsa_attention.py:1495-1675``, "full-chain" path) together with its cross-layer
reuse of top-k indices (``easyvolcap/official_vggt/models/aggregator.py:390-423, 681-694``: a layer listed in
``reuse_topk_source_by_layer`` takes the indices its source layer selected and skips its own indexer).
With a ``source_layout`` the indexer stage is the coarse-to-fine selection (``geoweave_b200.coarse_to_fine``): 2x2-pooled
patch cells are ranked and the kept cells expanded to tokens (the reference's ``source_downsample_enabled``,
``dsa_attention.py:1534-1556``).
The output projection, MLP and residuals around it are row-local model code and stay with the caller.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from . import _lib
from .custom_flash_attn.sparse_index_flash_attn import sparse_index_flash_attn_inference_func
from .coarse_to_fine import SourceLayout, select_topk_coarse_to_fine
from .custom_indexer.sparse_topk_indexer import fused_score_topk, indexer_workspace_bytes
from .front_end import HEAD_DIM, FrontEndParams, project_qkv_and_indexer


class SparseGlobalAttentionLayer:
    """``layer(x, pos)`` -> ``(out [B,N,H*64], idx int32 [B,N,k])``.

    ``reuse_topk_indices``: indices selected by an earlier layer; the indexer is skipped (its projections are
    still part of the one GEMM, as in the reference, whose fused weight is cached per layer).
    ``use_cuda_graph``: the chain is captured once per (shape, dtype, reuse or not) and replayed; inputs are copied
    into the graph's own buffers and the results are views of buffers that the next call overwrites.
    ``source_layout``: select coarse-to-fine over this layout's pooled sources instead of over all tokens;
    ``pool_queries``: pool the queries too and give every token the list of its cell.
    """

    def __init__(self, params: FrontEndParams, topk: int, idx_scale: Optional[float] = None,
                 attn_scale: Optional[float] = None, use_cuda_graph: bool = False,
                 source_layout: Optional[SourceLayout] = None, pool_queries: bool = False):
        self.params = params
        self.source_layout = source_layout
        self.pool_queries = bool(pool_queries)
        self.topk = int(topk)
        self.idx_scale = float(idx_scale) if idx_scale is not None else HEAD_DIM ** -0.5
        self.attn_scale = float(attn_scale) if attn_scale is not None else HEAD_DIM ** -0.5
        self.use_cuda_graph = bool(use_cuda_graph)
        self._graphs: Dict[tuple, dict] = {}

    # the chain itself: every call only enqueues on the current stream
    def _chain(self, x, pos, reuse_idx, workspace=None):
        q, k, v, q_idx, k_idx, w = project_qkv_and_indexer(x, pos, self.params)
        if reuse_idx is None:
            with torch.inference_mode():
                if self.source_layout is not None:
                    idx = select_topk_coarse_to_fine(q_idx, k_idx, w, self.source_layout, min(self.topk, x.shape[1]),
                                                     self.idx_scale, workspace=workspace, pool_queries=self.pool_queries)
                else:
                    idx, _ = fused_score_topk(q_idx, k_idx, w, min(self.topk, x.shape[1]), self.idx_scale, return_scores=False,
                                              workspace=workspace)
        else:
            idx = reuse_idx
        out, _ = sparse_index_flash_attn_inference_func(q, k, v, idx, None, False, self.attn_scale)
        return out.reshape(x.shape[0], x.shape[1], -1), idx

    def __call__(self, x: torch.Tensor, pos: Optional[torch.Tensor] = None,
                 reuse_topk_indices: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        _lib.require_cuda(x)
        if reuse_topk_indices is not None:
            if reuse_topk_indices.dtype != torch.int32 or tuple(reuse_topk_indices.shape[:2]) != tuple(x.shape[:2]):
                raise ValueError("reuse_topk_indices must be int32 [B,N,k] for this input")
            reuse_topk_indices = reuse_topk_indices.contiguous()
        if not self.use_cuda_graph:
            return self._chain(x, pos, reuse_topk_indices)
        key = (tuple(x.shape), x.dtype, x.device.index, pos is not None,
               None if reuse_topk_indices is None else tuple(reuse_topk_indices.shape))
        g = self._graphs.get(key)
        if g is None:
            g = self._capture(x, pos, reuse_topk_indices)
            self._graphs[key] = g
        g["x"].copy_(x)
        if pos is not None:
            g["pos"].copy_(pos)
        if reuse_topk_indices is not None:
            g["idx_in"].copy_(reuse_topk_indices)
        g["graph"].replay()
        return g["out"], g["idx"]

    def _capture(self, x, pos, reuse_idx):
        st = {"x": x.clone(), "pos": None if pos is None else pos.to(torch.int64).clone(),
              "idx_in": None if reuse_idx is None else reuse_idx.clone(), "ws": None}
        if reuse_idx is None:
            # the graph records raw pointers, so it owns its indexer workspace: a buffer from the shared cache could
            # be replaced (a larger shape, clear_runtime_cache) while the graph is still replayed
            B, N = x.shape[:2]
            if self.source_layout is not None:
                lay = self.source_layout
                nbytes = indexer_workspace_bytes(B, N, lay.source_len, self.params.idx_heads, HEAD_DIM, lay.kept_sources(min(self.topk, N)))
            else:
                nbytes = indexer_workspace_bytes(B, N, N, self.params.idx_heads, HEAD_DIM, min(self.topk, N))
            st["ws"] = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=x.device)
        side = torch.cuda.Stream(device=x.device)
        side.wait_stream(torch.cuda.current_stream(x.device))
        with torch.cuda.stream(side):  # first-use set-up of the library and of torch happens outside the capture
            self._chain(st["x"], st["pos"], st["idx_in"], st["ws"])
        torch.cuda.current_stream(x.device).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out, idx = self._chain(st["x"], st["pos"], st["idx_in"], st["ws"])
        st.update(graph=graph, out=out, idx=idx)
        return st
