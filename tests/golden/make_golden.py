"""Generate the golden fixtures in this directory by RUNNING THE REFERENCE on CPU.

Run once, in a container that has the reference checkout (it is not needed afterwards and never at test time):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py --reference /path/to/GeoWeave

What is recorded per case (all produced by reference code, nothing by this repository's oracle):

* ``scores``      LightningIndexer._compute_scores                      (easyvolcap/official_vggt/layers/indexer.py:383-428)
* ``ref_idx``     LightningIndexer.select_topk_projected (torch.topk)   (indexer.py:521-604) -- tie order unspecified
* ``blk_idx``     sparse_topk_indexer_func on CPU (block-wise streaming) (easyvolcap/utils/custom_indexer/sparse_topk_indexer.py:2188)
* ``tie_idx``     stable descending sort of ``scores`` (ties -> lower index), sorted ascending
* ``out``/``attn`` DSAAttention._sparse_attention                        (easyvolcap/official_vggt/layers/dsa_attention.py:4731-4753)
* ``out_pad``/``attn_sum_pad`` the reference test-suite's gathered-softmax formula with -1 padding
                  (tests/sparse_index_flash_attn_tests.py:47-71)

Inputs are bf16-representable and stored as their upper 16 bits (key suffix ``:bf16``); ``tests/golden/__init__.py`` decodes them.
"""
import argparse
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bf16_round(x):
    return x.to(torch.bfloat16).to(torch.float32)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a checkout of the reference project")
    args = ap.parse_args()
    sys.dont_write_bytecode = True
    sys.path[:0] = [os.path.join(HERE, "_stubs"), args.reference]

    from easyvolcap.utils.base_utils import dotdict
    from easyvolcap.official_vggt.layers.dsa_attention import DSAAttention
    from easyvolcap.utils.custom_indexer import sparse_topk_indexer_func

    def attention_module(heads, dim_head, hi, di, topk):
        cfg = dotdict(enabled=True, n_heads=hi, head_dim=di, topk=topk, use_topk_kernel=False,
                      use_sparse_flash_attn=False, score_dtype="float32")
        return DSAAttention(heads * dim_head, num_heads=heads, qk_norm=True, indexer_cfg=cfg).eval()

    # the reference test-suite's padded formula (a script, loaded by path; only the pure function is used)
    spec = importlib.util.spec_from_file_location(
        "_ref_sparse_tests", os.path.join(args.reference, "tests", "sparse_index_flash_attn_tests.py"))
    ref_tests = importlib.util.module_from_spec(spec)
    try:
        spec.loader.exec_module(ref_tests)
        padded_formula = ref_tests._reference_sparse_attn
    except Exception as exc:  # pragma: no cover
        print("could not import the reference test module:", repr(exc))
        padded_formula = None

    out = {}
    g = torch.Generator().manual_seed(20261125)

    def indexer_case(name, T, S, Hi, Di, k, kind):
        if kind.startswith("int"):
            q = torch.randint(-3, 4, (1, T, Hi, Di), generator=g).float()
            kk = torch.randint(-3, 4, (1, S, Hi, Di), generator=g).float()
            w = torch.randint(0, 9, (1, S, Hi), generator=g).float() / 8.0
        else:
            q = bf16_round(torch.randn(1, T, Hi, Di, generator=g))
            kk = bf16_round(torch.randn(1, S, Hi, Di, generator=g))
            if kind == "negw":
                w = bf16_round(torch.randn(1, S, Hi, generator=g))
            else:
                w = bf16_round(torch.rand(1, S, Hi, generator=g))
        if kind.endswith("ties"):
            n_dup = max(1, S // 10)
            dst = torch.randperm(S, generator=g)[:n_dup]
            src = torch.randint(0, S, (n_dup,), generator=g)
            kk[0, dst] = kk[0, src]
            w[0, dst] = w[0, src]
        m = attention_module(4, 64, Hi, Di, k)
        with torch.no_grad():
            scores = m.indexer._compute_scores(q, kk, w, None)
            ref_idx, ref_sc = m.indexer.select_topk_projected(q, kk, w, topk=k, return_scores=True)
            blk_idx, _ = sparse_topk_indexer_func(q, kk, w, q.new_empty(0), k, float(m.indexer.scale), 256, 0)
        kk_eff = min(k, S)
        tie_idx = torch.sort(torch.sort(scores, dim=-1, descending=True, stable=True).indices[..., :kk_eff], -1).values
        out.update({
            f"{name}.q_idx": q.numpy(), f"{name}.k_idx": kk.numpy(), f"{name}.w": w.numpy(),
            f"{name}.k": np.int64(k), f"{name}.scale": np.float64(float(m.indexer.scale)),
            f"{name}.scores": scores.numpy(), f"{name}.ref_idx": ref_idx.to(torch.int32).numpy(),
            f"{name}.blk_idx": blk_idx.to(torch.int32).numpy(), f"{name}.tie_idx": tie_idx.to(torch.int32).numpy(),
        })
        print(name, "scores", tuple(scores.shape), "rows where torch.topk set == tie-exact set:",
              int((torch.sort(ref_idx, -1).values == tie_idx).all(-1).sum()), "/", T)

    indexer_case("idx_int", 300, 300, 4, 64, 64, "int")
    indexer_case("idx_int_ties", 200, 333, 4, 64, 100, "int_ties")
    indexer_case("idx_bf16", 200, 520, 4, 64, 96, "bf16")
    indexer_case("idx_bf16_ties", 130, 400, 4, 64, 128, "bf16_ties")
    indexer_case("idx_negw", 64, 257, 4, 64, 32, "negw")
    indexer_case("idx_kgeS", 33, 40, 4, 64, 64, "bf16")
    indexer_case("idx_h2d32", 50, 190, 2, 32, 16, "bf16")

    def attention_case(name, B, T, S, H, D, K, pad):
        q = bf16_round(torch.randn(B, H, T, D, generator=g))
        k = bf16_round(torch.randn(B, H, S, D, generator=g))
        v = bf16_round(torch.randn(B, H, S, D, generator=g))
        idx = torch.stack([torch.stack([torch.randperm(S, generator=g)[:K] for _ in range(T)]) for _ in range(B)])
        m = attention_module(H, D, 4, 64, K)
        with torch.no_grad():
            o, attn = m._sparse_attention(q, k, v, idx, None)  # [B,H,T,D], [B,H,T,K]
        rec = {
            f"{name}.q": q.permute(0, 2, 1, 3).contiguous().numpy(), f"{name}.k": k.permute(0, 2, 1, 3).contiguous().numpy(),
            f"{name}.v": v.permute(0, 2, 1, 3).contiguous().numpy(), f"{name}.idx": idx.to(torch.int32).numpy(),
            f"{name}.scale": np.float64(float(m.scale) if hasattr(m, "scale") else D ** -0.5),
            f"{name}.out": o.permute(0, 2, 1, 3).contiguous().numpy(), f"{name}.attn_sum": attn.sum(1).numpy(),
        }
        if pad and padded_formula is not None:
            idx_p = idx.clone().to(torch.int32)
            for b in range(B):
                for t in range(T):
                    n_valid = int(torch.randint(max(1, K // 2), K + 1, (1,), generator=g))
                    idx_p[b, t, n_valid:] = -1
            with torch.no_grad():
                o_p, as_p = padded_formula(q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3), idx_p,
                                           softmax_scale=D ** -0.5)
            rec.update({f"{name}.idx_pad": idx_p.numpy(), f"{name}.out_pad": o_p.contiguous().numpy(),
                        f"{name}.attn_sum_pad": as_p.numpy()})
        out.update(rec)
        print(name, "out", tuple(o.shape))

    # the padded formula of the reference test-suite assumes self-attention (T == S)
    attention_case("attn_h4", 1, 128, 128, 4, 64, 48, True)
    attention_case("attn_h16", 2, 48, 48, 16, 64, 32, True)
    attention_case("attn_tnes", 1, 24, 120, 16, 64, 96, False)
    attention_case("attn_d128", 1, 24, 90, 8, 128, 40, False)
    attention_case("attn_d32", 1, 70, 70, 8, 32, 33, True)

    # inputs are bf16-representable: keep their upper 16 bits only (suffix ":bf16"), which halves the file
    packed = {}
    for key, val in out.items():
        leaf = key.split(".")[-1]
        if leaf in ("q_idx", "k_idx", "w", "q", "k", "v") and val.dtype == np.float32:
            bits = val.view(np.uint32)
            assert not (bits & 0xFFFF).any(), key
            packed[key + ":bf16"] = (bits >> 16).astype(np.uint16)
        else:
            packed[key] = val
    path = os.path.join(HERE, "reference_cpu.npz")
    np.savez_compressed(path, **packed)
    print("wrote", path, os.path.getsize(path) // 1024, "KiB")


if __name__ == "__main__":
    main()
