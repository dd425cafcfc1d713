"""Sparse-index flash attention, forward and backward -- same call signatures as the reference module
``easyvolcap/utils/custom_flash_attn/sparse_index_flash_attn.py`` (entry points at :3139, :3168, :3286, :3370).

Every function runs the hand-written sm_100a kernel behind ``gw_sparse_attn_fwd``; there is no Triton and
no CPU path.  Arguments the reference accepts but rejects on its sparse path (``bias``, ``causal``; its
kernel asserts ``BIAS_TYPE == 'none'`` and ``not IS_CAUSAL`` at :199,:204) raise ``NotImplementedError``.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from .. import _lib
from .._lists import group_by_key

__all__ = [
    "sparse_index_flash_attn_inference_func",
    "sparse_index_flash_attn_inference_bhtd_func",
    "sparse_index_flash_attn_func",
    "sparse_index_flash_attn_bhtd_func",
    "dense_index_flash_attn_func",
    "sparse_index_flash_attn_value_gate_bhtd_func",
    "sparse_attention_forward",
    "sparse_attention_backward",
]


def sparse_attention_forward(q, k, v, kv_positions, softmax_scale=None, return_attn=False, return_lse=False,
                             layout="bthd"):
    """Shared implementation.  ``layout`` names the order of q/k/v dims: 'bthd' or 'bhtd'.

    Returns ``(o, attn_sum or None, lse or None)``; ``o`` is a fresh contiguous tensor shaped like ``q``
    (the reference allocates ``torch.empty(q.shape)`` too, :2070), ``lse`` is fp32 ``[B,H,T]``.
    """
    if layout not in ("bthd", "bhtd"):
        raise ValueError(f"Unsupported q_layout: {layout}")
    dev = _lib.require_cuda(q, k, v, kv_positions)
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("q, k, v must be 4-D")
    if not (q.dtype == k.dtype == v.dtype):
        raise TypeError("All tensors must have the same type")
    if kv_positions.dtype != torch.int32:
        raise TypeError("kv_positions must be int32")
    q, k, v = [x if x.stride(-1) == 1 else x.contiguous() for x in (q, k, v)]
    if layout == "bthd":
        B, T, H, D = q.shape
        S = k.shape[1]
        expect = (B, S, H, D)
        dims = (0, 1, 2)
    else:
        B, H, T, D = q.shape
        S = k.shape[2]
        expect = (B, H, S, D)
        dims = (0, 2, 1)
    if tuple(k.shape) != expect or tuple(v.shape) != expect:
        raise ValueError(f"k/v shape {tuple(k.shape)}/{tuple(v.shape)} does not match q {tuple(q.shape)}")
    if D > 128:
        raise ValueError("head dimensions up to 128 are supported")
    if kv_positions.dim() != 3 or kv_positions.shape[0] != B or kv_positions.shape[1] != T:
        raise ValueError(f"kv_positions must be [B,T,K], got {tuple(kv_positions.shape)}")
    kv_positions = kv_positions.contiguous()
    K = kv_positions.shape[-1]
    es = q.element_size()

    def usable(x):  # the kernel gathers with 16-byte bulk copies
        return x.data_ptr() % 16 == 0 and all((x.stride(d) * es) % 16 == 0 for d in dims)

    q, k, v = [x if usable(x) else x.contiguous() for x in (q, k, v)]
    scale = float(softmax_scale) if softmax_scale else 1.0 / math.sqrt(D)
    o = torch.empty(q.shape, device=dev, dtype=q.dtype)
    want_lse = return_lse or return_attn
    lse = torch.empty((B, H, T), device=dev, dtype=torch.float32) if want_lse else None
    attn_sum = torch.empty((B, T, K), device=dev, dtype=torch.float32) if return_attn else None
    if T == 0 or K == 0:
        if attn_sum is not None:
            attn_sum.zero_()
        return o.zero_(), attn_sum, lse
    strides = lambda x: _lib.i64x3([x.stride(d) for d in dims])
    lib = _lib.load()
    with torch.cuda.device(dev):
        rc = lib.gw_sparse_attn_fwd(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), kv_positions.data_ptr(), _lib.dtype_code(q), B, T, S, H, D, K,
            strides(q), strides(k), strides(v), scale, o.data_ptr(), strides(o), _lib.ptr(lse), _lib.ptr(attn_sum),
            _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev))
    _lib.check(rc, "gw_sparse_attn_fwd")
    if _lib.debug_enabled():
        _lib.check_status(dev)
    return o, attn_sum, (lse if return_lse else None)


def _reject(bias, causal):
    if bias is not None:
        raise NotImplementedError("bias is not supported on the sparse-index path (the reference asserts BIAS_TYPE == 'none')")
    if causal:
        raise NotImplementedError("causal masking is not supported on the sparse-index path (the reference asserts it off)")


@torch.inference_mode()
def sparse_index_flash_attn_inference_func(q, k, v, kv_positions, bias: Optional[torch.Tensor] = None, causal: bool = False,
                                           softmax_scale: Optional[float] = None,
                                           return_attn: bool = False) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """q, k, v: ``[B,T,H,D]`` / ``[B,S,H,D]``; kv_positions int32 ``[B,T,K]``.  Returns ``(o, attn_sum | None)``."""
    _reject(bias, causal)
    o, attn_sum, _ = sparse_attention_forward(q, k, v, kv_positions, softmax_scale, return_attn, False, "bthd")
    return o, attn_sum


@torch.inference_mode()
def sparse_index_flash_attn_inference_bhtd_func(q, k, v, kv_positions, bias: Optional[torch.Tensor] = None,
                                                causal: bool = False, softmax_scale: Optional[float] = None,
                                                return_attn: bool = False) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """As above with q, k, v kept in ``[B,H,T,D]`` layout (gathered head by head, no transpose copy)."""
    _reject(bias, causal)
    o, attn_sum, _ = sparse_attention_forward(q, k, v, kv_positions, softmax_scale, return_attn, False, "bhtd")
    return o, attn_sum


def sparse_attention_backward(q, k, v, kv_positions, o, lse, d_out, d_attn_sum, softmax_scale):
    """Gradients of the forward for ``[B,T,H,D]`` / ``[B,S,H,D]`` tensors: ``(dq, dk, dv)`` of the inputs' dtype.

    ``d_attn_sum`` (fp32 ``[B,T,K]`` or None) is the gradient arriving through the forward's second result.  The sums
    over the queries that selected a key run in a fixed order (the index lists are stably sorted by key first, here
    with ``torch.sort``), so the result is reproducible; there are no floating-point atomics in the kernels."""
    dev = _lib.require_cuda(q, k, v, kv_positions, o, d_out)
    B, T, H, D = q.shape
    S = k.shape[1]
    K = kv_positions.shape[-1]
    if D != 64 or H > 32:
        raise NotImplementedError("the backward kernels are built for head_dim 64 and at most 32 heads")
    q, k, v, o, d_out = [x.contiguous() for x in (q, k, v, o, d_out.to(q.dtype))]
    kv_positions = kv_positions.contiguous()
    lse = lse.contiguous()
    if d_attn_sum is not None:
        d_attn_sum = d_attn_sum.to(torch.float32).contiguous()
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    if T == 0 or K == 0:
        return dq.zero_(), dk.zero_(), dv.zero_()
    order, start = group_by_key(kv_positions, S)  # (query, slot) pairs grouped by key, in a fixed order
    lib = _lib.load()
    ws = torch.empty(int(lib.gw_sparse_attn_bwd_workspace_bytes(B, T, H, K)), dtype=torch.uint8, device=dev)
    scale = float(softmax_scale) if softmax_scale else 1.0 / math.sqrt(D)
    with torch.cuda.device(dev):
        rc = lib.gw_sparse_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), kv_positions.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                    d_out.data_ptr(), _lib.ptr(d_attn_sum), order.data_ptr(), start.data_ptr(), _lib.dtype_code(q),
                                    B, T, S, H, D, K, scale, dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), ws.data_ptr(), ws.numel(),
                                    _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev))
    _lib.check(rc, "gw_sparse_attn_bwd")
    if _lib.debug_enabled():
        _lib.check_status(dev)
    return dq, dk, dv


class _SparseIndexFlashAttn(torch.autograd.Function):
    """The reference's ``SparseIndexFlashAttnFunc`` / ``SparseIndexFlashAttnBhtdFunc`` (:3196-3370): forward returns
    ``(o, attn_sum)``, backward returns the gradients of q, k and v (both results may carry a gradient)."""

    @staticmethod
    def forward(ctx, q, k, v, kv_positions, softmax_scale, layout):
        o, attn_sum, lse = sparse_attention_forward(q, k, v, kv_positions, softmax_scale, True, True, layout)
        ctx.save_for_backward(q, k, v, kv_positions, o, lse)
        ctx.set_materialize_grads(False)  # a result the loss does not use arrives as None, not as a tensor of zeros
        ctx.softmax_scale = softmax_scale
        ctx.layout = layout
        return o, attn_sum

    @staticmethod
    def backward(ctx, d_o, d_attn_sum):
        q, k, v, kv_positions, o, lse = ctx.saved_tensors
        to_bthd = (lambda x: x.transpose(1, 2)) if ctx.layout == "bhtd" else (lambda x: x)
        if d_o is None:
            d_o = torch.zeros_like(o)
        dq, dk, dv = sparse_attention_backward(to_bthd(q), to_bthd(k), to_bthd(v), kv_positions, to_bthd(o), lse, to_bthd(d_o),
                                               d_attn_sum, ctx.softmax_scale)
        return to_bthd(dq), to_bthd(dk), to_bthd(dv), None, None, None


def _wants_grad(*tensors):
    return torch.is_grad_enabled() and any(t.requires_grad for t in tensors)


def sparse_index_flash_attn_func(q, k, v, kv_positions, bias=None, causal=False, softmax_scale=None):
    """The reference's autograd entry (``SparseIndexFlashAttnFunc.apply``): returns ``(o, attn_sum)`` with ``attn_sum``
    fp32 ``[B,T,K]``; differentiable in q, k and v."""
    _reject(bias, causal)
    if _wants_grad(q, k, v):
        return _SparseIndexFlashAttn.apply(q, k, v, kv_positions, softmax_scale, "bthd")
    with torch.no_grad():
        o, attn_sum, _ = sparse_attention_forward(q, k, v, kv_positions, softmax_scale, True, False, "bthd")
    return o, attn_sum


def sparse_index_flash_attn_bhtd_func(q, k, v, kv_positions, bias=None, causal=False, softmax_scale=None):
    _reject(bias, causal)
    if _wants_grad(q, k, v):
        return _SparseIndexFlashAttn.apply(q, k, v, kv_positions, softmax_scale, "bhtd")
    with torch.no_grad():
        o, attn_sum, _ = sparse_attention_forward(q, k, v, kv_positions, softmax_scale, True, False, "bhtd")
    return o, attn_sum


def dense_index_flash_attn_func(q, k, v, bias=None, causal=False, softmax_scale=None):
    """Dense attention through the sparse kernel (every key listed for every query), as the reference's
    ``dense_index_flash_attn_func`` (:3121) does.  Meant for small problems and tests."""
    B, T = q.shape[0], q.shape[1]
    S = k.shape[1]
    pos = torch.arange(S, device=q.device, dtype=torch.int32).view(1, 1, S).expand(B, T, S).contiguous()
    return sparse_index_flash_attn_func(q, k, v, pos, bias, causal, softmax_scale)


def sparse_index_flash_attn_value_gate_bhtd_func(*args, **kwargs):
    raise NotImplementedError("the value-gate variant is a training-time option of the reference and is not part of "
                              "this library (both published presets keep it off)")
