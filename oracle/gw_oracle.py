"""CPU restatement of the reference's torch-backend math for the sparse top-k global-attention path.

TEST INFRASTRUCTURE ONLY -- the product path never imports this file and has no CPU fallback.

Parity status: PINNED.  ``tests/test_oracle_golden.py`` checks every function below against
fixtures produced by running the reference's own code on CPU (``tests/golden/make_golden.py``).

What each function follows (paths are relative to the reference project):

* ``indexer_scores``      easyvolcap/official_vggt/layers/indexer.py:430-466 (``_compute_score_chunk``):
                          ``einsum('bthd,bshd->bths') * scale -> relu -> * w[s,h] -> sum over heads`` in fp32.
* ``topk_tie_exact``      easyvolcap/official_vggt/layers/indexer.py:601-603 (``scores.topk(k, sorted=False)``),
                          made deterministic: exact top-k, equal scores keep the LOWER key index.  The
                          reference leaves tie order unspecified (its tests accept either index,
                          tests/indexer_projected_tests.py:95-96), so this rule is a strict refinement.
* ``merge_two_topk``      easyvolcap/utils/custom_indexer/csrc/merge_two_topk_kernel.cu:24-74
                          (sort the union of two k-lists by score, keep k), same tie rule.
* ``sparse_attention``    easyvolcap/official_vggt/layers/dsa_attention.py:4731-4753 (``_sparse_attention``:
                          gather K -> q.K^T*scale -> softmax over the k selected keys -> gather V -> p.V) with the
                          padding rule of the kernel path, easyvolcap/utils/custom_flash_attn/
                          sparse_index_flash_attn.py:208-218 (index < 0 or >= S contributes nothing), and the
                          ``attn_sum``/LSE side outputs of :375-458 and :250-252.
* ``source_layout`` / ``coarse_topk`` / ``pool_sources`` / ``expand_sources``
                          the coarse-to-fine selector of easyvolcap/official_vggt/layers/dsa_attention.py:3069-3258,
                          3328-3375, 3386-3543, 4079-4128 (factor 2, "legacy" strategy: rank pooled 2x2 cells, expand the
                          kept cells round-robin to tokens).
* ``audit_topk``          the acceptance rule for a kernel that computes its own fp32 scores in a different
                          summation order: any index it picks that the oracle did not must sit within a
                          rounding bound of the oracle's k-th score.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np
import torch

__all__ = [
    "indexer_scores",
    "topk_tie_exact",
    "indexer_topk",
    "merge_two_topk",
    "sparse_attention",
    "score_error_bound",
    "audit_topk",
    "source_layout",
    "token_source",
    "coarse_topk",
    "pool_sources",
    "expand_sources",
]


def _f32(x) -> torch.Tensor:
    if isinstance(x, np.ndarray):
        x = torch.from_numpy(x)
    return x.detach().to("cpu", torch.float32)


def indexer_scores(q_idx, k_idx, w, scale: Optional[float] = None, row_chunk: int = 1024) -> torch.Tensor:
    """fp32 scores ``[B,T,S]`` from ``q_idx [B,T,Hi,Di]``, ``k_idx [B,S,Hi,Di]``, ``w [B,S,Hi]``.

    Inputs of any float dtype are widened to fp32 first (the torch backend of the reference forces
    ``score_dtype=float32``, geoweave/inference.py:56-58).  Query rows are independent, so the work is done in
    row chunks to keep the ``[B,rows,Hi,S]`` intermediate small.
    """
    q, k, w = _f32(q_idx), _f32(k_idx), _f32(w)
    B, T, Hi, Di = q.shape
    S = k.shape[1]
    if scale is None:
        scale = 1.0 / math.sqrt(Di)
    w_by_head = w.permute(0, 2, 1)  # [B,Hi,S]
    out = torch.empty((B, T, S), dtype=torch.float32)
    for t0 in range(0, T, row_chunk):
        t1 = min(T, t0 + row_chunk)
        hs = torch.einsum("bthd,bshd->bths", q[:, t0:t1], k) * scale
        hs = torch.relu(hs)
        hs = hs * w_by_head.unsqueeze(1)
        out[:, t0:t1] = hs.sum(dim=2, dtype=torch.float32)
    return out


def topk_tie_exact(scores, k: int) -> torch.Tensor:
    """Exact top-k per row of ``scores [..., C]``; ties keep the lower column.  Returns int32 ``[..., k]``
    sorted ascending by column index (the order itself carries no meaning: the reference returns its
    indices unsorted and consumers only gather with them)."""
    s = _f32(scores)
    k = min(int(k), s.shape[-1])
    # -0.0 and +0.0 compare equal, so the stable sort treats them as a tie (lower index wins).
    order = torch.sort(s, dim=-1, descending=True, stable=True).indices[..., :k]
    return torch.sort(order, dim=-1).values.to(torch.int32)


def indexer_topk(q_idx, k_idx, w, k: int, scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Stage 1+2 in one call: returns (indices int32 ``[B,T,k]`` ascending, their fp32 scores)."""
    sc = indexer_scores(q_idx, k_idx, w, scale)
    idx = topk_tie_exact(sc, k)
    return idx, sc.gather(-1, idx.long())


def merge_two_topk(a_scores, a_idx, b_scores, b_idx, k: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Keep the best k of the union of two per-row candidate lists ``[..., ka]`` and ``[..., kb]``.

    Order is (score descending, key index ascending); returned lists are sorted ascending by index.
    Negative indices mark empty slots and always lose.
    """
    a_s, b_s = _f32(a_scores), _f32(b_scores)
    a_i = torch.as_tensor(a_idx).to(torch.int64)
    b_i = torch.as_tensor(b_idx).to(torch.int64)
    if k is None:
        k = a_s.shape[-1]
    s = torch.cat([a_s, b_s], -1)
    i = torch.cat([a_i, b_i], -1)
    s = torch.where(i < 0, torch.full_like(s, -float("inf")), s)
    # sort by index first, then stably by score: equal scores end up in ascending index order.
    by_idx = torch.sort(torch.where(i < 0, torch.full_like(i, 2**62), i), dim=-1, stable=True)
    s1 = s.gather(-1, by_idx.indices)
    i1 = i.gather(-1, by_idx.indices)
    by_score = torch.sort(s1, dim=-1, descending=True, stable=True)
    top_i = i1.gather(-1, by_score.indices[..., :k])
    top_s = by_score.values[..., :k]
    fin = torch.sort(top_i, dim=-1, stable=True)
    return top_s.gather(-1, fin.indices), fin.values.to(torch.int32)


def sparse_attention(
    q, k, v, kv_positions, scale: Optional[float] = None, row_chunk: int = 256
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Attention of every query over only its selected keys, fp32 math.

    ``q [B,T,H,D]``, ``k,v [B,S,H,D]``, ``kv_positions [B,T,K]`` (all heads of a query share one list).
    Returns ``(out [B,T,H,D] fp32, lse [B,H,T] fp32 natural log, attn_sum [B,T,K] fp32 = sum over heads of p)``.
    A row whose positions are all padding yields zeros and ``lse = -inf``.
    """
    q, k, v = _f32(q), _f32(k), _f32(v)
    pos = torch.as_tensor(kv_positions).to("cpu", torch.int64)
    B, T, H, D = q.shape
    S = k.shape[1]
    K = pos.shape[-1]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    out = torch.zeros((B, T, H, D), dtype=torch.float32)
    lse = torch.full((B, H, T), -float("inf"), dtype=torch.float32)
    attn_sum = torch.zeros((B, T, K), dtype=torch.float32)
    kh = k.permute(0, 2, 1, 3)  # [B,H,S,D]
    vh = v.permute(0, 2, 1, 3)
    for b in range(B):
        for t0 in range(0, T, row_chunk):
            t1 = min(T, t0 + row_chunk)
            p_ = pos[b, t0:t1]  # [r,K]
            valid = (p_ >= 0) & (p_ < S)
            safe = torch.where(valid, p_, torch.zeros_like(p_))
            k_sel = kh[b][:, safe]  # [H,r,K,D]
            sc = torch.matmul(q[b, t0:t1].permute(1, 0, 2).unsqueeze(-2), k_sel.transpose(-1, -2)).squeeze(-2) * scale
            sc = sc.masked_fill(~valid.unsqueeze(0), -float("inf"))  # [H,r,K]
            row_lse = torch.logsumexp(sc, dim=-1)  # [H,r]
            attn = torch.softmax(sc, dim=-1)
            attn = torch.where(valid.unsqueeze(0), attn, torch.zeros_like(attn))
            attn = torch.nan_to_num(attn, nan=0.0)  # all-padding rows
            v_sel = vh[b][:, safe]
            o = torch.matmul(attn.unsqueeze(-2), v_sel).squeeze(-2)  # [H,r,D]
            out[b, t0:t1] = o.permute(1, 0, 2)
            lse[b, :, t0:t1] = row_lse
            attn_sum[b, t0:t1] = attn.sum(0)
    return out, lse, attn_sum


def score_error_bound(q_idx, k_idx, w, rows: torch.Tensor, cols: torch.Tensor, scale: float, c: float = 64.0):
    """Worst-case |difference| between two fp32 evaluations of score[row, col] that differ only in summation
    order: ``c * 2^-24 * scale * sum_h |w[s,h]| * sum_d |q[t,h,d] * k[s,h,d]|`` (products of bf16 values are exact
    in fp32; only the additions round).  ``rows``/``cols`` are 1-D index tensors of equal length (batch 0)."""
    q, k, w = _f32(q_idx)[0], _f32(k_idx)[0], _f32(w)[0]
    prod = (q[rows].abs() * k[cols].abs()).sum(-1)  # [n,Hi]
    return c * 2.0**-24 * scale * (prod * w[cols].abs()).sum(-1)


def audit_topk(idx_test, scores_oracle, k: int, q_idx=None, k_idx=None, w=None, scale: float = 0.125, c: float = 64.0):
    """Compare index sets chosen from scores computed elsewhere against the oracle's choice on ``scores_oracle``.

    Returns a dict: rows, rows_equal, swapped (entries picked that the oracle did not pick), unexplained
    (swapped entries farther from the oracle's k-th score than the rounding bound; must be 0), max_gap.
    With ``q_idx/k_idx/w`` omitted the bound is 0, i.e. only exact ties can be swapped.
    """
    sc = _f32(scores_oracle)
    if sc.dim() == 2:
        sc = sc.unsqueeze(0)
    it = torch.as_tensor(idx_test).to("cpu", torch.int64)
    if it.dim() == 2:
        it = it.unsqueeze(0)
    ref = topk_tie_exact(sc, k).long()
    test_sorted = torch.sort(it, -1).values
    equal_rows = (test_sorted == ref).all(-1)
    res = dict(rows=int(equal_rows.numel()), rows_equal=int(equal_rows.sum()), swapped=0, unexplained=0, max_gap=0.0,
               duplicates=0, out_of_range=0)
    S = sc.shape[-1]
    res["out_of_range"] = int(((it < 0) | (it >= S)).sum())
    res["duplicates"] = int((test_sorted[..., 1:] == test_sorted[..., :-1]).sum())
    if bool(equal_rows.all()) or res["out_of_range"]:
        return res
    bad_b, bad_t = torch.nonzero(~equal_rows, as_tuple=True)
    for b, t in zip(bad_b.tolist(), bad_t.tolist()):
        row = sc[b, t]
        kth = row[ref[b, t]].min()
        in_ref = torch.zeros(S, dtype=torch.bool)
        in_ref[ref[b, t]] = True
        extra = test_sorted[b, t][~in_ref[test_sorted[b, t]]]
        if extra.numel() == 0:
            continue
        gap = (kth - row[extra]).abs()
        if q_idx is not None and b == 0:
            bound = score_error_bound(q_idx, k_idx, w, torch.full_like(extra, t), extra, scale, c)
            # the k-th element itself carries the same kind of error
            bound = bound + score_error_bound(q_idx, k_idx, w, torch.tensor([t]), ref[b, t][row[ref[b, t]].argmin()].view(1), scale, c)
        else:
            bound = torch.zeros_like(gap)
        res["swapped"] += int(extra.numel())
        res["unexplained"] += int((gap > bound).sum())
        res["max_gap"] = max(res["max_gap"], float(gap.max()))
    return res


def reference_cpu_path(q_idx, k_idx, w, q, k, v, topk: int, idx_scale: float, attn_scale: float, rows: slice):
    """The op sequence the reference's ``--device cpu --backend torch`` path executes for a slice of query rows
    (geoweave/inference.py:56-60): dense fp32 scores (indexer.py:452-455), ``torch.topk(sorted=False)``
    (indexer.py:602), then gather / matmul / softmax / matmul (dsa_attention.py:4731-4753).  Used as the timed
    CPU arm of the benchmark; query rows are independent, so a slice of rows with all keys resident costs
    exactly its share of the full problem.  Layouts: q_idx ``[1,T,Hi,Di]``, q/k/v ``[1,H,N,D]`` (the
    reference's), fp32."""
    qi = q_idx[:, rows]
    hs = torch.einsum("bthd,bshd->bths", qi, k_idx) * idx_scale
    hs = torch.relu(hs)
    hs = hs * w.permute(0, 2, 1).unsqueeze(1)
    scores = hs.sum(dim=2, dtype=torch.float32)
    idx = scores.topk(min(topk, scores.shape[-1]), dim=-1, sorted=False)[1]
    B, H, S, D = k.shape
    T = idx.shape[1]

    def gather(x):
        flat = idx[:, None].expand(B, H, T, idx.shape[2]).reshape(B * H, -1)
        return x.reshape(B * H, S, D).gather(1, flat.unsqueeze(-1).expand(-1, -1, D)).reshape(B, H, T, -1, D)

    k_sel = gather(k)
    sc = torch.matmul(q[:, :, rows].unsqueeze(-2), k_sel.transpose(-1, -2)).squeeze(-2) * attn_scale
    del k_sel
    attn = sc.softmax(dim=-1)
    out = torch.matmul(attn.unsqueeze(-2), gather(v)).squeeze(-2)
    return out, idx


# ---------------------------------------------------------------------------------------------
# projection front-end: what DSAAttention.forward does between its fused linear layer and the operator calls
# ---------------------------------------------------------------------------------------------
def _layer_norm(x, weight, bias, eps):
    """LayerNorm over the last dimension (biased variance), as torch.nn.LayerNorm."""
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    y = (x - mean) / torch.sqrt(var + eps)
    if weight is not None:
        y = y * weight + bias
    return y


def _rope_2d(tokens, pos, cos_tab, sin_tab):
    """2-D rotary embedding of ``tokens [B,N,heads,D]`` at integer positions ``pos [B,N,2]`` (y, x).

    The first half of the head dimension is rotated by the y position, the second by the x position; inside a
    half of width F the pairs are (j, j + F/2) and both members use table column j mod F/2 (the tables hold
    cat(angles, angles)) -- official_vggt/layers/rope.py:117-188.
    """
    D = tokens.shape[-1]
    F_ = D // 2
    out = torch.empty_like(tokens)
    for half, axis in ((slice(0, F_), 0), (slice(F_, D), 1)):
        t = tokens[..., half]
        cos = cos_tab[pos[..., axis]][:, :, None, :]  # [B,N,1,F]
        sin = sin_tab[pos[..., axis]][:, :, None, :]
        rot = torch.cat((-t[..., F_ // 2:], t[..., : F_ // 2]), dim=-1)
        out[..., half] = t * cos + rot * sin
    return out


def project_front_end(fused, pos, cos_tab, sin_tab, heads, head_dim, idx_heads, idx_dim, q_norm=None, k_norm=None,
                      idx_k_norm=None):
    """From the output of the fused linear layer to the six operator inputs, fp32 math.

    ``fused [B,N,3*H*D + 2*Hi*Di + Hi]`` holds, per token, [q | k | v | idx_q | idx_k | idx_w] in that order
    (dsa_attention.py:545-600: the weights of qkv, q_proj, k_proj, w_proj are concatenated; qkv itself is
    [3][H][D], :229-232).  q and k get LayerNorm over the head dimension, then the 2-D rotary embedding (:4935-4941);
    idx_k gets its LayerNorm, idx_q and idx_k the same rotary embedding, idx_w is passed through (indexer.py:302-328).
    Each ``*_norm`` is ``(weight, bias, eps)`` or None.  Returns ``q, k, v [B,N,H,D]``, ``q_idx, k_idx [B,N,Hi,Di]``,
    ``w [B,N,Hi]``, all fp32.
    """
    f = _f32(fused)
    B, N, _ = f.shape
    H, D, Hi, Di = heads, head_dim, idx_heads, idx_dim
    pos = torch.as_tensor(pos).to(torch.int64)
    cos_tab, sin_tab = _f32(cos_tab), _f32(sin_tab)
    qkv = f[..., : 3 * H * D].reshape(B, N, 3, H, D)
    o = 3 * H * D
    iq = f[..., o: o + Hi * Di].reshape(B, N, Hi, Di)
    ik = f[..., o + Hi * Di: o + 2 * Hi * Di].reshape(B, N, Hi, Di)
    w = f[..., o + 2 * Hi * Di: o + 2 * Hi * Di + Hi].clone()
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2].clone()

    def norm(x, prm):
        return x if prm is None else _layer_norm(x, _f32(prm[0]), _f32(prm[1]), float(prm[2]))

    q = _rope_2d(norm(q, q_norm), pos, cos_tab, sin_tab)
    k = _rope_2d(norm(k, k_norm), pos, cos_tab, sin_tab)
    iq = _rope_2d(iq, pos, cos_tab, sin_tab)
    ik = _rope_2d(norm(ik, idx_k_norm), pos, cos_tab, sin_tab)
    return q, k, v, iq, ik, w


# ---------------------------------------------------------------------------------------------------------------------
# Coarse-to-fine selection (pooled sources), factor 2, round-robin expansion -- the reference's "legacy" strategy
# ---------------------------------------------------------------------------------------------------------------------
def source_layout(tokens_per_view: int, num_views: int, patch_start: int, grid_h: int, grid_w: int, factor: int = 2) -> dict:
    """The list of "sources" the coarse stage ranks (dsa_attention.py:3069-3258, ``_get_source_downsample_layout``
    without representative points): first every view's special tokens, then every patch token outside the pooled
    region (``y >= pooled_h or x >= pooled_w``; view-major, row-major), then the ``factor x factor`` cells (view-major,
    row-major), each with its fine tokens in row-major order.  ``source_to_fine`` is int64 ``[L, factor*factor]`` with
    -1 for missing slots."""
    assert tokens_per_view - patch_start == grid_h * grid_w
    pooled_h, pooled_w = grid_h // factor * factor, grid_w // factor * factor
    coarse_h, coarse_w = pooled_h // factor, pooled_w // factor
    rows = []
    for v in range(num_views):
        rows += [[v * tokens_per_view + s] for s in range(patch_start)]
    special = len(rows)
    for v in range(num_views):
        base = v * tokens_per_view + patch_start
        rows += [[base + y * grid_w + x] for y in range(grid_h) for x in range(grid_w) if not (y < pooled_h and x < pooled_w)]
    edge = len(rows) - special
    for v in range(num_views):
        base = v * tokens_per_view + patch_start
        for cy in range(coarse_h):
            for cx in range(coarse_w):
                rows.append([base + (cy * factor + yy) * grid_w + cx * factor + xx for yy in range(factor) for xx in range(factor)])
    width = factor * factor
    table = torch.full((len(rows), width), -1, dtype=torch.int64)
    for r, toks in enumerate(rows):
        table[r, : len(toks)] = torch.tensor(toks)
    coarse = len(rows) - special - edge
    mapped = special + edge + coarse * width
    return dict(source_to_fine=table, source_len=len(rows), special_count=special, edge_count=edge, coarse_count=coarse,
                avg_expand=mapped / len(rows), non_special_source_len=len(rows) - special,
                non_special_avg_expand=(mapped - special) / max(len(rows) - special, 1), factor=factor)


def token_source(layout: dict) -> torch.Tensor:
    """int64 [N]: the source each token belongs to (``fine_to_source_row``, dsa_attention.py:3186-3196); with pooled
    queries every token takes the list selected for that source (:3996-4017)."""
    table = layout["source_to_fine"]
    out = torch.full((int(table.max()) + 1,), -1, dtype=torch.int64)
    rows = torch.arange(table.shape[0]).view(-1, 1).expand_as(table)
    out[table[table >= 0]] = rows[table >= 0]
    return out


def coarse_topk(layout: dict, topk: int, ratio: float = 1.1) -> int:
    """How many sources the coarse stage keeps (dsa_attention.py:3328-3375 for the legacy strategy with
    ``source_downsample_coarse_topk = 0``)."""
    m = int(math.ceil(topk / max(layout["avg_expand"], 1.0) * max(ratio, 1.0)))
    special = min(layout["special_count"], topk)
    if 0 < special < topk and m < special and layout["non_special_source_len"] > 0:
        rem = int(math.ceil((topk - special) / max(layout["non_special_avg_expand"], 1.0) * max(ratio, 1.0)))
        m = max(m, special + max(rem, 1))
    return min(max(m, 1), layout["source_len"])


def pool_sources(k_idx, w, layout: dict):
    """Keys and weights of the sources (dsa_attention.py:3386-3543): a special or edge source is its token, a cell is
    the mean of its tokens (``avg_pool2d``), in fp32 here.  ``k_idx [B,N,Hi,Di]``, ``w [B,N,Hi]`` -> ``[B,L,Hi,Di]``,
    ``[B,L,Hi]``."""
    table = layout["source_to_fine"]
    valid = table >= 0
    safe = table.clamp_min(0)
    kf, wf = _f32(k_idx), _f32(w)
    cnt = valid.sum(-1).to(torch.float32)
    ks = (kf[:, safe] * valid[None, :, :, None, None]).sum(2) / cnt[None, :, None, None]
    ws = (wf[:, safe] * valid[None, :, :, None]).sum(2) / cnt[None, :, None]
    return ks, ws


def expand_sources(coarse_idx, layout: dict, topk: int, fine_len: int, pad_window: int = 64) -> torch.Tensor:
    """From each query's ORDERED list of sources to ``min(topk, fine_len)`` token indices (dsa_attention.py:4079-4128,
    round-robin form): slot 0 of every listed source in list order, then slot 1 of every source that has one, and so
    on; cut to the target length; a list that is too short is padded by cycling over its last ``pad_window`` entries."""
    table = layout["source_to_fine"]
    B, T, m = coarse_idx.shape
    target = min(int(topk), int(fine_len))
    out = torch.empty((B, T, target), dtype=torch.int64)
    for b in range(B):
        for t in range(T):
            blocks = table[coarse_idx[b, t].long()]                      # [m, width]
            flat = blocks.t().reshape(-1)                                # slot-major
            toks = flat[flat >= 0][:target]
            n = max(int(toks.numel()), 1)
            if toks.numel() < target:
                win = min(n, max(1, min(int(pad_window), target)))
                start = n - win
                pad = torch.tensor([int(toks[start + (i % win)]) for i in range(target - toks.numel())], dtype=torch.int64)
                toks = torch.cat([toks, pad])
            out[b, t] = toks
    return out
