"""Golden fixtures for the projection front-end (the step in front of the indexer and the sparse attention),
made by RUNNING THE REFERENCE modules on CPU.

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden_frontend.py --reference /path/to/GeoWeave

Per case (all tensors produced by reference code):

* ``x``, ``pos``                   the layer input and the (y, x) token positions
* ``weight``, ``bias``, ``splits`` DSAAttention._get_fused_proj_params  (official_vggt/layers/dsa_attention.py:545-585)
* ``fused``                        F.linear(x, weight, bias) as in _project_qkv_and_indexer_fused (:587-600)
* ``q``, ``k``, ``v``              qkv -> _project_attention_qkv_from_flat -> q_norm / k_norm -> rope, as
                                   DSAAttention.forward does (:4933-4941), returned token-major [B,N,H,D]
* ``q_idx``, ``k_idx``, ``w``      LightningIndexer.project  (official_vggt/layers/indexer.py:302-328)
* ``cos``, ``sin``                 RotaryPositionEmbedding2D._compute_frequency_components (layers/rope.py:84-115)
* the LayerNorm parameters of q_norm, k_norm and the indexer's k_norm

``*_bf16`` cases run the same modules converted to bfloat16 on a bfloat16 input (values stored as fp32).
"""
import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a checkout of the reference project")
    args = ap.parse_args()
    sys.dont_write_bytecode = True
    sys.path[:0] = [os.path.join(HERE, "_stubs"), args.reference]

    import torch.nn.functional as F
    from easyvolcap.utils.base_utils import dotdict
    from easyvolcap.official_vggt.layers.dsa_attention import DSAAttention
    from easyvolcap.official_vggt.layers.rope import PositionGetter, RotaryPositionEmbedding2D

    out = {}
    g = torch.Generator().manual_seed(20261126)

    def case(name, heads, views, gh, gw, n_special, dtype, eps):
        dim = heads * 64
        cfg = dotdict(enabled=True, n_heads=4, head_dim=64, topk=16, use_topk_kernel=False, use_sparse_flash_attn=False,
                      score_dtype="float32" if dtype == torch.float32 else "bfloat16", qk_norm=True)
        norm = (lambda d: torch.nn.LayerNorm(d, eps=eps))
        rope = RotaryPositionEmbedding2D(frequency=100)
        m = DSAAttention(dim, num_heads=heads, qkv_bias=True, qk_norm=True, norm_layer=norm, rope=rope, indexer_cfg=cfg).eval()
        with torch.no_grad():  # the default initialisation (unit LayerNorm, zero w_proj) would hide mistakes
            for p in m.parameters():
                p.copy_(torch.randn(p.shape, generator=g) * (0.5 if p.dim() == 1 else dim ** -0.5))
            for ln in (m.q_norm, m.k_norm, m.indexer.k_norm):
                if isinstance(ln, torch.nn.LayerNorm):
                    ln.weight.add_(1.0)
        n_tok = n_special + gh * gw
        pos = PositionGetter()(views, gh, gw, torch.device("cpu")) + 1
        pos = torch.cat([torch.zeros(views, n_special, 2, dtype=pos.dtype), pos], 1).view(1, views * n_tok, 2)
        x = torch.randn(1, views * n_tok, dim, generator=g)
        if dtype != torch.float32:
            m = m.to(dtype)
            x = x.to(dtype)
        with torch.no_grad():
            weight, bias, splits = m._get_fused_proj_params(cache=False)
            fused = F.linear(x, weight, bias)
            qkv = m.qkv(x)
            q, k, v = m._project_attention_qkv_from_flat(qkv, 1, x.shape[1])
            q, k = m.q_norm(q), m.k_norm(k)
            q, k = m.rope(q, pos), m.rope(k, pos)
            q_idx, k_idx, w = m.indexer.project(x, pos)
            cos, sin = rope._compute_frequency_components(32, int(pos.max()) + 1, x.device, x.dtype)
        f32 = lambda t: t.detach().float().contiguous().numpy()
        rec = dict(x=f32(x), pos=pos.numpy().astype(np.int64), weight=f32(weight), bias=f32(bias), splits=np.asarray(splits, np.int64),
                   fused=f32(fused), q=f32(q.permute(0, 2, 1, 3)), k=f32(k.permute(0, 2, 1, 3)), v=f32(v.permute(0, 2, 1, 3)),
                   q_idx=f32(q_idx), k_idx=f32(k_idx), w=f32(w), cos=f32(cos), sin=f32(sin), eps=np.float64(eps),
                   heads=np.int64(heads), q_norm_w=f32(m.q_norm.weight), q_norm_b=f32(m.q_norm.bias),
                   k_norm_w=f32(m.k_norm.weight), k_norm_b=f32(m.k_norm.bias),
                   ik_norm_w=f32(m.indexer.k_norm.weight), ik_norm_b=f32(m.indexer.k_norm.bias),
                   ik_norm_eps=np.float64(m.indexer.k_norm.eps))
        for key, val in rec.items():
            out[f"{name}.{key}"] = val
        print(name, "tokens", x.shape[1], "fused", tuple(fused.shape), "q", tuple(q.shape), "q_idx", tuple(q_idx.shape), q_idx.dtype)

    case("fe_f32", 2, 3, 4, 6, 5, torch.float32, 1e-5)      # VGGT-like: 5 special tokens per view, LayerNorm eps 1e-5
    case("fe_bf16", 2, 3, 4, 6, 5, torch.bfloat16, 1e-5)
    case("fe_pi3_bf16", 3, 2, 5, 3, 5, torch.bfloat16, 1e-6)  # Pi3-like: eps 1e-6
    path = os.path.join(HERE, "reference_frontend.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path) // 1024, "KiB")


if __name__ == "__main__":
    main()
