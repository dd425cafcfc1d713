"""The reference's own caller on the GPU, with this library installed under its operator names.

One global-attention block of the reference (``DSABlock`` for VGGT, ``DSABlockRope`` for Pi3; seeded trunc-normal
weights, bf16) runs the same tokens twice: once with the reference's torch backend
(``use_topk_kernel=False, use_sparse_flash_attn=False, score_dtype=float32`` -- ``geoweave/inference.py:56-60``),
once after ``geoweave_b200.install()`` with the kernel backend switched on, so that
``LightningIndexer.select_topk_projected`` (``official_vggt/layers/indexer.py:565-599``) and the dispatch in
``DSAAttention.forward`` (``official_vggt/layers/dsa_attention.py:5275-5400``) call this library unchanged.

Checked: the selected indices are an exact top-k of the oracle's scores on the block's own projections (no
unexplained entry, no duplicate), and the attention output, the attention module's output and the block's
output agree with the torch backend within 2e-2.  Needs the staged reference (``baseline/stage_reference.py``).
"""
import pytest
import torch

from baseline import ref_harness as rh
from oracle import gw_oracle as orc
from tests.gpu_util import dev

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not rh.available(), reason="the reference is not staged under baseline/_ref")]

VIEWS, TOPK = 4, 1024  # 4 views: N = 4164 (VGGT) / 3128 (Pi3), the reference's CPU-runnable size


class _Calls:
    """Counts calls of the rebound operator names inside the reference's caller modules."""

    def __init__(self, monkeypatch):
        import importlib

        self.n = {}
        for mod_name, names in (
            ("easyvolcap.official_vggt.layers.indexer", ("sparse_topk_indexer_func", "sparse_topk_indexer_inference_func")),
            ("easyvolcap.official_vggt.layers.dsa_attention", ("sparse_index_flash_attn_func", "sparse_index_flash_attn_inference_func",
                                                             "sparse_index_flash_attn_inference_bhtd_func")),
        ):
            mod = importlib.import_module(mod_name)
            for name in names:
                fn = getattr(mod, name)
                assert fn.__module__.startswith("geoweave_b200."), f"{mod_name}.{name} is not this library's function"
                monkeypatch.setattr(mod, name, self._wrap(name, fn))

    def _wrap(self, name, fn):
        def counted(*a, **k):
            self.n[name] = self.n.get(name, 0) + 1
            return fn(*a, **k)

        return counted


def _proj_input_hook(block, store):
    return block.attn.proj.register_forward_pre_hook(lambda _m, args: store.__setitem__("o", args[0].detach()))


@pytest.mark.parametrize("model,entries", [
    ("vggt", "inference"),   # VGGT_INDEXER_TOPK_INFER_DIRECT=1 + sparse_flash_disable_attn_sum: the two inference entries
    ("vggt", "autograd"),    # defaults: sparse_topk_indexer_func + sparse_index_flash_attn_func (returns attn_sum)
    ("pi3", "inference"),
])
def test_reference_block_kernel_backend_matches_its_torch_backend(model, entries, monkeypatch):
    import geoweave_b200

    rh.enable_import()
    blk = rh.build_block(model, TOPK, seed=3, device=dev(), dtype=torch.bfloat16)
    x, pos = rh.make_inputs(model, VIEWS, seed=3, device=dev(), dtype=torch.bfloat16)
    N = x.shape[1]

    # --- the reference's torch backend (fp32 scores and attention over the block's bf16 projections)
    got = {}
    hook = _proj_input_hook(blk, got)
    rh.set_backend(blk, model, VIEWS, "torch", TOPK)
    y_ref, cap_ref = rh.run_block(blk, model, x, pos)
    o_ref = got.pop("o").float()
    assert cap_ref.topk_indices.dtype == torch.int64 and tuple(cap_ref.topk_indices.shape) == (1, N, TOPK)
    torch.cuda.empty_cache()

    # --- the same block with this library bound to the reference's operator names
    patched = geoweave_b200.install()
    try:
        assert any(p.endswith("indexer.sparse_topk_indexer_func") for p in patched)
        calls = _Calls(monkeypatch)
        if entries == "inference":
            monkeypatch.setenv("VGGT_INDEXER_TOPK_INFER_DIRECT", "1")
        rh.set_backend(blk, model, VIEWS, "kernel", TOPK)
        if entries == "autograd":
            blk.indexer_state.sparse_flash_disable_attn_sum = False
        y_ker, cap_ker = rh.run_block(blk, model, x, pos)
        geoweave_b200.check_status()
    finally:
        hook.remove()
        geoweave_b200.uninstall()
    o_ker = got.pop("o").float()
    if entries == "inference":
        assert calls.n == {"sparse_topk_indexer_inference_func": 1, "sparse_index_flash_attn_inference_func": 1}, calls.n
    else:
        assert calls.n == {"sparse_topk_indexer_func": 1, "sparse_index_flash_attn_func": 1}, calls.n
    idx_ker = cap_ker.topk_indices
    assert tuple(idx_ker.shape) == (1, N, TOPK)

    # --- indices: exact top-k of the oracle's scores on the block's own indexer projections (sampled rows)
    q, k, v, q_idx, k_idx, w = [t.cpu() for t in rh.operator_inputs(blk, cap_ker.attn_in, pos)]
    rows = torch.arange(0, N, 13)
    scores = orc.indexer_scores(q_idx[:, rows], k_idx, w, 0.125)
    for name, idx in (("kernel", idx_ker), ("torch", cap_ref.topk_indices)):
        res = orc.audit_topk(idx[:, rows.to(idx.device)], scores, TOPK, q_idx[:, rows], k_idx, w, 0.125)
        assert res["out_of_range"] == 0 and res["duplicates"] == 0 and res["unexplained"] == 0, (name, res)
    full = torch.sort(idx_ker.long(), -1).values
    assert int(full.min()) >= 0 and int(full.max()) < N and bool((full[..., 1:] != full[..., :-1]).all())
    same = (full == torch.sort(cap_ref.topk_indices, -1).values).all(-1).float().mean().item()
    assert same >= 0.98, f"only {same:.4f} of the rows select the same set as the torch backend"

    # --- outputs against the torch backend: attention (before the output projection), attention module, block
    assert (o_ker - o_ref).abs().max().item() <= 2e-2
    assert (cap_ker.attn_out.float() - cap_ref.attn_out.float()).abs().max().item() <= 2e-2
    assert (y_ker.float() - y_ref.float()).abs().max().item() <= 2e-2
    # and the attention against the oracle on the very indices the kernel backend selected
    ref_o, _, _ = orc.sparse_attention(q[:, rows], k, v, idx_ker[:, rows.to(dev())].cpu(), 0.125)
    assert (o_ker.view(1, N, 16, 64)[:, rows.to(dev())].cpu() - ref_o).abs().max().item() <= 2e-2


def test_operator_inputs_of_the_reference_block_have_the_statistics_the_bench_workload_uses():
    """`bench.py --workload vggt32_proj` draws its operator inputs from this harness; pin what it relies on:
    w is about 1 +- 0.64 (the w_proj bias of 1 dominates), k_idx is LayerNorm'd (unit scale), q_idx is not."""
    rh.enable_import()
    blk = rh.build_block("vggt", TOPK, seed=5, device=dev(), dtype=torch.bfloat16)
    x, pos = rh.make_inputs("vggt", 2, seed=5, device=dev(), dtype=torch.bfloat16)
    with torch.no_grad():
        q, k, v, q_idx, k_idx, w = rh.operator_inputs(blk, blk.norm1(x), pos)
    assert q.dtype == torch.bfloat16 and tuple(q.shape) == (1, x.shape[1], 16, 64) and q.is_contiguous()
    assert 0.9 < w.float().mean().item() < 1.1 and 0.5 < w.float().std().item() < 0.8
    assert 0.9 < k_idx.float().std().item() < 1.1 and 0.5 < q_idx.float().std().item() < 0.8
