"""Projection front-end of a sparse global layer: the step between the layer's linear projections and the two
operators.  Mirrors what ``DSAAttention`` does there
(``easyvolcap/official_vggt/layers/dsa_attention.py:545-627`` fused projection, ``:229-232`` qkv split,
``:4935-4941`` q/k LayerNorm and rotary embedding, ``:5309-5315`` the ``.contiguous()`` transposes) together
with ``LightningIndexer.project`` (``easyvolcap/official_vggt/layers/indexer.py:302-328``).

The linear layer itself stays a library GEMM (``torch.nn.functional.linear``, one call for the concatenated
weights, as the reference's fused variant does); everything after it is one CUDA kernel
(``gw_project_epilogue``) that writes q, k, v, q_idx, k_idx and w token-major and contiguous, ready for
``sparse_topk_indexer_*`` and ``sparse_index_flash_attn_*``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _lib

HEAD_DIM = 64


@dataclass
class FrontEndParams:
    """Parameters of one layer, gathered once (the reference caches the same concatenation, ``:545-585``).

    ``weight [3*H*64 + 2*Hi*64 + Hi, dim]`` / ``bias`` are the rows of qkv, indexer.q_proj, indexer.k_proj and
    indexer.w_proj in that order.  A LayerNorm is ``(weight, bias, eps)`` with fp32 vectors of 64, or None.
    ``cos`` / ``sin`` fp32 ``[positions, 32]`` are the tables of the rotary module, or None for no rotary embedding.
    """
    weight: torch.Tensor
    bias: Optional[torch.Tensor]
    heads: int
    idx_heads: int
    q_norm: Optional[Tuple[torch.Tensor, torch.Tensor, float]] = None
    k_norm: Optional[Tuple[torch.Tensor, torch.Tensor, float]] = None
    idx_k_norm: Optional[Tuple[torch.Tensor, torch.Tensor, float]] = None
    cos: Optional[torch.Tensor] = None
    sin: Optional[torch.Tensor] = None


def rope_tables(max_position: int, device, dtype: torch.dtype, frequency: float = 100.0, feature_dim: int = HEAD_DIM // 2):
    """The cos / sin tables of ``RotaryPositionEmbedding2D`` (``layers/rope.py:84-115``) for positions
    ``0..max_position-1``: the angles are rounded to ``dtype`` before and after the trigonometry, exactly as the
    reference does for tokens of that dtype; returned as fp32 for the kernel."""
    exponents = torch.arange(0, feature_dim, 2, device=device).float() / feature_dim
    inv_freq = 1.0 / (frequency ** exponents)
    positions = torch.arange(max_position, device=device, dtype=inv_freq.dtype)
    angles = torch.einsum("i,j->ij", positions, inv_freq).to(dtype)
    angles = torch.cat((angles, angles), dim=-1)
    return angles.cos().to(dtype).float().contiguous(), angles.sin().to(dtype).float().contiguous()


def _norm_tuple(ln) -> Optional[Tuple[torch.Tensor, torch.Tensor, float]]:
    if not isinstance(ln, torch.nn.LayerNorm):
        return None
    w = ln.weight if ln.weight is not None else torch.ones(ln.normalized_shape, device="cpu")
    b = ln.bias if ln.bias is not None else torch.zeros_like(w)
    return w.detach().float().contiguous(), b.detach().float().contiguous(), float(ln.eps)


def params_from_module(attn, max_position: int, dtype: torch.dtype) -> FrontEndParams:
    """Collect the parameters from a reference ``DSAAttention`` (or any object with the same attributes: ``qkv``,
    ``q_norm``, ``k_norm``, ``rope``, ``num_heads`` and ``indexer`` with ``q_proj``, ``k_proj``, ``w_proj``, ``k_norm``,
    ``n_heads``)."""
    idx = attn.indexer
    linears = (attn.qkv, idx.q_proj, idx.k_proj, idx.w_proj)
    weight = torch.cat([lin.weight for lin in linears], dim=0).detach()
    bias = torch.cat([lin.bias if lin.bias is not None else lin.weight.new_zeros(lin.out_features) for lin in linears]).detach()
    cos = sin = None
    if getattr(attn, "rope", None) is not None:
        cos, sin = rope_tables(max_position, weight.device, dtype, float(attn.rope.base_frequency))
    return FrontEndParams(weight, bias, int(attn.num_heads), int(idx.n_heads), _norm_tuple(attn.q_norm), _norm_tuple(attn.k_norm),
                          _norm_tuple(idx.k_norm), cos, sin)


def project_epilogue(fused: torch.Tensor, pos: Optional[torch.Tensor], prm: FrontEndParams):
    """``fused [B,N,3*H*64 + 2*Hi*64 + Hi]`` (the linear layer's output) -> ``q, k, v [B,N,H,64]``,
    ``q_idx, k_idx [B,N,Hi,64]``, ``w [B,N,Hi]`` of the same dtype."""
    lib = _lib.load()
    dev = _lib.require_cuda(fused)
    if fused.dim() != 3:
        raise ValueError(f"fused must be [B,N,C], got shape={tuple(fused.shape)}")
    B, N, C = fused.shape
    H, Hi = prm.heads, prm.idx_heads
    width = 3 * H * HEAD_DIM + 2 * Hi * HEAD_DIM + Hi
    if C != width:
        raise ValueError(f"fused has {C} columns, the layer needs {width} (heads={H}, indexer heads={Hi}, head dim 64)")
    if not fused.is_contiguous():
        fused = fused.contiguous()
    ld = C
    if (C * fused.element_size()) % 8 != 0:  # the kernel reads rows in 8- or 16-byte pieces (an odd number of indexer heads)
        ld = C + (-C) % 8
        fused = F.pad(fused, (0, ld - C))
    if pos is not None:
        if prm.cos is None:
            raise ValueError("positions given but the parameters hold no rotary tables")
        if tuple(pos.shape) != (B, N, 2):
            raise ValueError(f"pos must be [B,N,2], got shape={tuple(pos.shape)}")
        pos = pos.to(device=dev, dtype=torch.int64).contiguous()
    out = [torch.empty((B, N, H, HEAD_DIM), device=dev, dtype=fused.dtype) for _ in range(3)]
    out += [torch.empty((B, N, Hi, HEAD_DIM), device=dev, dtype=fused.dtype) for _ in range(2)]
    out.append(torch.empty((B, N, Hi), device=dev, dtype=fused.dtype))

    # parameters that live elsewhere are brought to the device here and kept alive until the launch is enqueued
    norms = [None if n is None else (n[0].to(dev, torch.float32).contiguous(), n[1].to(dev, torch.float32).contiguous(), float(n[2]))
             for n in (prm.q_norm, prm.k_norm, prm.idx_k_norm)]
    qn, kn, ikn = [(None, None, 0.0) if n is None else (n[0].data_ptr(), n[1].data_ptr(), n[2]) for n in norms]
    cos = prm.cos.to(dev, torch.float32).contiguous() if pos is not None else None
    sin = prm.sin.to(dev, torch.float32).contiguous() if pos is not None else None
    with torch.cuda.device(dev):
        rc = lib.gw_project_epilogue(fused.data_ptr(), _lib.dtype_code(fused), B * N, ld, H, HEAD_DIM, Hi, HEAD_DIM, _lib.ptr(pos),
                                     _lib.ptr(cos), _lib.ptr(sin), 0 if cos is None else cos.shape[0], qn[0], qn[1], qn[2],
                                     kn[0], kn[1], kn[2], ikn[0], ikn[1], ikn[2], *[t.data_ptr() for t in out],
                                     _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev))
    _lib.check(rc, "gw_project_epilogue")
    del norms, cos, sin
    return tuple(out)


def project_fused(x: torch.Tensor, pos: Optional[torch.Tensor], prm: FrontEndParams):
    """Layer input ``x [B,N,dim]`` (bf16 / fp16, ``dim`` a multiple of 64) -> the six operator inputs in ONE kernel: the
    projection GEMM on the tcgen05 tensor cores with bias, LayerNorm, rotary embedding and the token-major stores in
    its epilogue.  The raw product ``[q | k | v | idx_q | idx_k | idx_w]`` never reaches memory."""
    lib = _lib.load()
    dev = _lib.require_cuda(x)
    if x.dim() != 3:
        raise ValueError(f"x must be [B,N,dim], got shape={tuple(x.shape)}")
    if x.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError("the fused projection takes bfloat16 or float16 tokens (fp32: project_epilogue after a library GEMM)")
    B, N, dim = x.shape
    H, Hi = prm.heads, prm.idx_heads
    width = 3 * H * HEAD_DIM + 2 * Hi * HEAD_DIM + Hi
    if tuple(prm.weight.shape) != (width, dim):
        raise ValueError(f"weight must be [{width}, {dim}], got {tuple(prm.weight.shape)}")
    if dim % 64 != 0:
        raise _lib.GeoWeaveError(-2, "the fused projection needs a model width that is a multiple of 64")
    x = x.contiguous()
    weight = prm.weight.to(dev, x.dtype).contiguous()
    bias = None if prm.bias is None else prm.bias.to(dev, x.dtype).contiguous()
    if pos is not None:
        if prm.cos is None:
            raise ValueError("positions given but the parameters hold no rotary tables")
        if tuple(pos.shape) != (B, N, 2):
            raise ValueError(f"pos must be [B,N,2], got shape={tuple(pos.shape)}")
        pos = pos.to(device=dev, dtype=torch.int64).contiguous()
    out = [torch.empty((B, N, H, HEAD_DIM), device=dev, dtype=x.dtype) for _ in range(3)]
    out += [torch.empty((B, N, Hi, HEAD_DIM), device=dev, dtype=x.dtype) for _ in range(2)]
    out.append(torch.empty((B, N, Hi), device=dev, dtype=x.dtype))
    norms = [None if n is None else (n[0].to(dev, torch.float32).contiguous(), n[1].to(dev, torch.float32).contiguous(), float(n[2]))
             for n in (prm.q_norm, prm.k_norm, prm.idx_k_norm)]
    qn, kn, ikn = [(None, None, 0.0) if n is None else (n[0].data_ptr(), n[1].data_ptr(), n[2]) for n in norms]
    cos = prm.cos.to(dev, torch.float32).contiguous() if pos is not None else None
    sin = prm.sin.to(dev, torch.float32).contiguous() if pos is not None else None
    with torch.cuda.device(dev):
        rc = lib.gw_project_fused(x.data_ptr(), weight.data_ptr(), _lib.ptr(bias), _lib.dtype_code(x), B * N, dim, H, HEAD_DIM, Hi,
                                  HEAD_DIM, _lib.ptr(pos), _lib.ptr(cos), _lib.ptr(sin), 0 if cos is None else cos.shape[0],
                                  qn[0], qn[1], qn[2], kn[0], kn[1], kn[2], ikn[0], ikn[1], ikn[2], *[t.data_ptr() for t in out],
                                  _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev))
    _lib.check(rc, "gw_project_fused")
    del norms, cos, sin, weight, bias
    return tuple(out)


def project_qkv_and_indexer(x: torch.Tensor, pos: Optional[torch.Tensor], prm: FrontEndParams):
    """Layer input ``x [B,N,dim]`` -> the six operator inputs.  16-bit tokens of a width that is a multiple of 64 go
    through the fused tensor-core kernel (``project_fused``); fp32 tokens, whose products the 16-bit tensor-core path
    would change, through a library GEMM followed by the epilogue kernel."""
    if x.dtype in (torch.bfloat16, torch.float16) and x.shape[-1] % 64 == 0:
        return project_fused(x, pos, prm)
    return project_epilogue(F.linear(x, prm.weight, prm.bias), pos, prm)
