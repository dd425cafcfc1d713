"""The reference project's OWN caller of the sparse global-attention path, built with seeded random weights.

Used by the GPU parity tests (torch backend of the reference vs this library's kernels installed under the
reference's operator names) and by ``bench.py --impl reference``.  It imports the staged copy of the reference
under ``baseline/_ref`` (``baseline/stage_reference.py``); nothing in the product package imports this file.

What is built is one global-attention block of the reference, exactly as its aggregator builds it:

* VGGT:  ``easyvolcap/official_vggt/layers/block.py:102-184`` (``DSABlock``; ``models/aggregator.py`` passes
  ``qkv_bias=True, proj_bias=True, ffn_bias=True, init_values=0.01, qk_norm=True,
  rope=RotaryPositionEmbedding2D(frequency=100)``), tokens per view = 5 special + 28 x 37 patches.
* Pi3:   ``aidi/third_party/pi3_training/pi3/models/layers/block.py:345-446`` (``DSABlockRope`` with
  ``norm_layer=LayerNorm(eps=1e-6)``, ``rope=RoPE2D(freq=100)``), tokens per view = 5 register + 21 x 37 patches.

The backend switch is the one of ``geoweave/inference.py:56-60``: the torch backend sets
``use_topk_kernel=False, use_sparse_flash_attn=False, score_dtype='float32'``; the kernel backend leaves the
preset's ``use_topk_kernel=True, use_sparse_flash_attn=True`` on.
"""
from __future__ import annotations

import os
import sys
from functools import partial
from typing import Optional, Tuple

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
STAGED = os.path.join(HERE, "_ref", "GeoWeave")
STUBS = os.path.join(HERE, "_ref", "_stubs")

GRIDS = {"vggt": (28, 37, 5), "pi3": (21, 37, 5)}  # patch rows, patch columns, special tokens per view


def available() -> bool:
    return os.path.isdir(os.path.join(STAGED, "easyvolcap"))


def enable_import() -> str:
    """Put the staged reference on ``sys.path`` (once).  Raises if it has not been staged."""
    if not available():
        raise FileNotFoundError(f"{STAGED} is missing: run `python baseline/stage_reference.py` where a checkout of the "
                                "reference exists")
    sys.dont_write_bytecode = True
    for p in (os.path.join(STAGED, "aidi", "third_party", "pi3_training"), STAGED, STUBS):
        if p not in sys.path:
            sys.path.insert(0, p)
    return STAGED


def tokens_per_view(model: str) -> int:
    gh, gw, special = GRIDS[model]
    return gh * gw + special


def indexer_cfg(topk: int = 1024, backend: str = "torch", kernel_dtype: str = "bfloat16"):
    """``indexer_cfg`` of the published presets (``geoweave/configs/{vggt,pi3}.json``) reduced to the keys the
    inference path reads, with the backend switch of ``geoweave/inference.py:56-60`` applied."""
    from easyvolcap.utils.base_utils import dotdict

    cfg = dotdict(enabled=True, n_heads=4, head_dim=64, topk=int(topk), eps=1e-6, detach_input=True, sparse_use_mask=False,
                  topk_block=256, use_topk_kernel=True, use_sparse_flash_attn=True, score_dtype=kernel_dtype,
                  sparse_flash_disable_attn_sum=True)
    if backend == "torch":
        cfg.update(use_topk_kernel=False, use_sparse_flash_attn=False, score_dtype="float32")
    elif backend != "kernel":
        raise ValueError(backend)
    return cfg


def set_backend(block, model: str, views: int, backend: str, topk: int = 1024, kernel_dtype: str = "bfloat16", **state) -> None:
    """Switch an existing block between the torch and the kernel backend (the same weights serve both).  ``state``:
    further keys of the per-layer indexer state, e.g. the selector options ``source_downsample_enabled`` /
    ``source_downsample_strategy`` / ``force_keep_special_tokens`` (``dsa_attention.py:3044-4277, 5042-5134``)."""
    from easyvolcap.utils.base_utils import dotdict

    cfg = indexer_cfg(topk, backend, kernel_dtype)
    gh, gw, special = GRIDS[model]
    block.attn.indexer_cfg = cfg
    block.attn.indexer.use_topk_kernel = bool(cfg.use_topk_kernel)
    block.attn.indexer.score_dtype = block.attn.indexer._parse_dtype(cfg.score_dtype)
    block.indexer_state = dotdict(cfg, enabled=True, warmup=False, sparse=True, compute_loss=False, layer_idx=9,
                                  tokens_per_view=tokens_per_view(model), num_views=int(views), patch_start_idx=special,
                                  patch_grid_height=gh, patch_grid_width=gw)
    block.indexer_state.update(state)
    block.return_indexer_loss = True  # as the aggregators do


def build_block(model: str = "vggt", topk: int = 1024, seed: int = 0, device="cpu", dtype=torch.float32):
    """One global-attention block of the reference with seeded weights: every Linear weight trunc-normal(std 0.02),
    biases zero except the indexer's ``w_proj`` bias, which keeps its initial value 1 (``indexer.py:63-68``);
    LayerNorm and layer-scale parameters as constructed."""
    enable_import()
    cfg = indexer_cfg(topk, "torch")
    if model == "vggt":
        from easyvolcap.official_vggt.layers.block import DSABlock
        from easyvolcap.official_vggt.layers.rope import RotaryPositionEmbedding2D

        blk = DSABlock(dim=1024, num_heads=16, mlp_ratio=4.0, qkv_bias=True, proj_bias=True, ffn_bias=True, init_values=0.01,
                       qk_norm=True, rope=RotaryPositionEmbedding2D(frequency=100), fused_attn=True, indexer_cfg=cfg)
    elif model == "pi3":
        from pi3.models.layers.block import DSABlockRope
        from pi3.models.layers.pos_embed import RoPE2D

        blk = DSABlockRope(dim=1024, num_heads=16, mlp_ratio=4.0, qkv_bias=True, proj_bias=True, ffn_bias=True,
                           norm_layer=partial(torch.nn.LayerNorm, eps=1e-6), init_values=0.01, qk_norm=True,
                           rope=RoPE2D(freq=100.0), indexer_cfg=cfg)
    else:
        raise ValueError(model)
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for name, mod in blk.named_modules():
            if isinstance(mod, torch.nn.Linear):
                wt = torch.empty(mod.weight.shape)
                torch.nn.init.trunc_normal_(wt, std=0.02, generator=g)
                mod.weight.copy_(wt)
                if mod.bias is not None and not name.endswith("w_proj"):
                    mod.bias.zero_()
    return blk.eval().to(device=device, dtype=dtype)


def make_inputs(model: str, views: int, seed: int = 0, device="cpu", dtype=torch.float32) -> Tuple[torch.Tensor, torch.Tensor]:
    """Tokens ``~N(0,1)`` ``[1, views*tokens_per_view, 1024]`` and their positions: patch (y, x) + 1, special tokens
    at (0, 0) (``official_vggt/models/aggregator.py:517-526``; Pi3 builds the same per view)."""
    gh, gw, special = GRIDS[model]
    g = torch.Generator().manual_seed(1000 + seed)
    n = views * (gh * gw + special)
    x = torch.randn(1, n, 1024, generator=g).to(device=device, dtype=dtype)
    ys, xs = torch.meshgrid(torch.arange(gh), torch.arange(gw), indexing="ij")
    grid = torch.stack([ys.reshape(-1), xs.reshape(-1)], -1) + 1
    pos = torch.cat([torch.zeros(special, 2, dtype=torch.long), grid]).repeat(views, 1).view(1, n, 2).to(device)
    return x, pos


class Captured:
    """What one forward of the block's attention module saw and produced."""
    attn_in: Optional[torch.Tensor] = None   # norm1(x): the attention module's input
    attn_out: Optional[torch.Tensor] = None  # its output (after the output projection)
    topk_indices: Optional[torch.Tensor] = None


def run_block(block, model: str, x: torch.Tensor, pos: torch.Tensor):
    """``(y, captured)``: the block's output and the attention module's input/output/selected indices."""
    cap = Captured()

    def pre(_mod, args, kwargs):
        cap.attn_in = args[0].detach()

    def post(_mod, _args, out):
        cap.attn_out = (out[0] if isinstance(out, tuple) else out).detach()

    h1 = block.attn.register_forward_pre_hook(pre, with_kwargs=True)
    h2 = block.attn.register_forward_hook(post)
    try:
        with torch.no_grad():
            y = block(x, pos=pos) if model == "vggt" else block(x, xpos=pos)
    finally:
        h1.remove()
        h2.remove()
    y = y[0] if isinstance(y, tuple) else y
    cap.topk_indices = block.attn.last_topk_indices
    return y, cap


def operator_inputs(block, attn_in: torch.Tensor, pos: torch.Tensor):
    """The six tensors that arrive at the operator boundary for this block input, made by the reference's own
    modules: ``q, k, v [1,N,16,64]`` (after q/k LayerNorm and rotary embedding, ``dsa_attention.py:4935-4941``) and
    ``q_idx, k_idx [1,N,4,64], w [1,N,4]`` (``LightningIndexer.project``, ``indexer.py:302-328``), in ``attn_in``'s dtype."""
    a = block.attn
    with torch.no_grad():
        B, N, _ = attn_in.shape
        q, k, v = a._project_attention_qkv_from_flat(a.qkv(attn_in), B, N)
        q, k = a.q_norm(q), a.k_norm(k)
        if a.rope is not None:
            q, k = a.rope(q, pos), a.rope(k, pos)
        saved = a.indexer.score_dtype
        a.indexer.score_dtype = None
        try:
            q_idx, k_idx, w = a.indexer.project(attn_in, pos=pos)
        finally:
            a.indexer.score_dtype = saved
    to_bthd = lambda t: t.transpose(1, 2).contiguous()
    return to_bthd(q), to_bthd(k), to_bthd(v), q_idx.contiguous(), k_idx.contiguous(), w.contiguous()
