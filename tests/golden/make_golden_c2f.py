"""Generate ``reference_c2f.npz`` by RUNNING THE REFERENCE's coarse-to-fine selector pieces on CPU.

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden_c2f.py --reference /path/to/GeoWeave

Recorded per case (all produced by reference code, ``easyvolcap/official_vggt/layers/dsa_attention.py``):

* ``table``, ``counts``   ``_get_source_downsample_layout`` (:3069-3258): source_to_fine and (source_len, special, edge,
                          coarse) -- plus ``coarse_topk`` from ``_resolve_source_downsample_coarse_topk`` (:3328-3375)
* ``src_k``, ``src_w``    ``_prepare_source_downsample_projected`` (:3386-3543) on seeded bf16-representable fp32 inputs
* ``fine``                ``_expand_source_downsample_chunk`` (:4079-4128) on seeded ordered lists of distinct sources
* ``coarse_q``, ``fine_to_row``  ``_prepare_query_downsample_chunk`` (:3925-3994) with the whole sequence as one chunk: the
                          pooled queries and, per token, the row of the list it takes (qk_sym_x2_broadcast)
"""
import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# (tokens_per_view, views, special tokens, grid_h, grid_w, topk, queries, record the pooled keys)
CASES = {
    "vggt2": (5 + 28 * 37, 2, 5, 28, 37, 256, 24, False),
    "pi3_3": (5 + 21 * 37, 3, 5, 21, 37, 1024, 8, False),
    "vggt1": (5 + 28 * 37, 1, 5, 28, 37, 128, 8, True),
    "odd": (2 + 5 * 7, 2, 2, 5, 7, 48, 20, True),       # an odd row and an odd column outside the pooled region
    "short": (1 + 4 * 4, 1, 1, 4, 4, 17, 9, True),      # every token is wanted: lists too short, padded by cycling
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    sys.dont_write_bytecode = True
    sys.path[:0] = [os.path.join(HERE, "_stubs"), args.reference]
    from easyvolcap.utils.base_utils import dotdict
    from easyvolcap.official_vggt.layers.dsa_attention import DSAAttention

    cfg = dotdict(enabled=True, n_heads=4, head_dim=64, topk=1024, use_topk_kernel=False, use_sparse_flash_attn=False,
                  score_dtype="float32")
    attn = DSAAttention(1024, num_heads=16, qk_norm=True, indexer_cfg=cfg).eval()
    out = {}
    for name, (tpv, views, special, gh, gw, topk, nq, pooled) in CASES.items():
        state = dotdict(tokens_per_view=tpv, num_views=views, patch_start_idx=special, patch_grid_height=gh, patch_grid_width=gw,
                        source_downsample_enabled=True, source_downsample_factor=2, source_downsample_strategy="legacy")
        n = tpv * views
        layout = attn._get_source_downsample_layout(state, n, torch.device("cpu"))
        m = attn._resolve_source_downsample_coarse_topk(state, layout, topk)
        out[f"{name}.table"] = layout.source_to_fine.numpy().astype(np.int32)
        out[f"{name}.counts"] = np.array([layout.source_len, layout.special_count, layout.edge_count, layout.coarse_count, m],
                                         dtype=np.int64)
        g = torch.Generator().manual_seed(len(name) + n)
        if pooled:
            k = torch.randn(1, n, 4, 64, generator=g).bfloat16().float()
            w = torch.randn(1, n, 4, generator=g).bfloat16().float()
            prep = attn._prepare_source_downsample_projected(k, w, state)
            out[f"{name}.k:bf16"] = (k.view(torch.int32).numpy() >> 16).astype(np.int16)
            out[f"{name}.w:bf16"] = (w.view(torch.int32).numpy() >> 16).astype(np.int16)
            out[f"{name}.src_k"] = prep.source_k.numpy()
            out[f"{name}.src_w"] = prep.source_w.numpy()
            qp = attn._prepare_query_downsample_chunk(k, layout, 0)     # the same tensor taken as queries, one chunk
            out[f"{name}.coarse_q"] = qp.coarse_q.numpy()
            out[f"{name}.fine_to_row"] = qp.fine_to_local_coarse_row.numpy().astype(np.int32)
        mm = min(m, layout.source_len)
        lists = torch.stack([torch.stack([torch.randperm(layout.source_len, generator=g)[:mm] for _ in range(nq)]) for _ in range(2)])
        fine = attn._expand_source_downsample_chunk(lists, layout, state, topk, n)
        out[f"{name}.lists"] = lists.numpy().astype(np.int32)
        out[f"{name}.fine"] = fine.numpy().astype(np.int32)
        print(name, "sources", layout.source_len, "kept", mm, "fine", tuple(fine.shape))
    np.savez_compressed(os.path.join(HERE, "reference_c2f.npz"), **out)


if __name__ == "__main__":
    main()
