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
        self.shapes = {}  # name -> [(shape of the first argument, shape of the second), ...]
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
            self.shapes.setdefault(name, []).append((tuple(a[0].shape), tuple(a[1].shape)))
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


@pytest.mark.parametrize("variant,state", [
    # coarse-to-fine selection: the indexer ranks 2x2-pooled source cells, the caller expands them to tokens
    ("pooled_sources", dict(source_downsample_enabled=True, source_downsample_factor=2, source_downsample_strategy="legacy")),
    # the same with pooled queries too, one list broadcast to the four queries of a cell
    ("pooled_queries_and_sources", dict(source_downsample_enabled=True, source_downsample_factor=2,
                                        source_downsample_strategy="qk_sym_x2_broadcast")),
    # forced tokens: every view's special tokens inside the top-k budget; the query's own view on top of the top-k
    ("special_tokens_in_budget", dict(force_keep_special_tokens=True, force_keep_special_in_topk_budget=True)),
    ("own_view_kept", dict(force_keep_self_view_tokens=True)),
])
def test_reference_selector_variants_run_on_this_library(variant, state, monkeypatch):
    """The reference's reductions of stage 1 (``dsa_attention.py:3044-4277, 4332-4360, 5042-5134``) are host logic of
    its caller around the same operator calls -- a coarse-to-fine selector that hands the indexer pooled keys (S < N) or
    pooled queries and keys, and forced special / own-view tokens merged with the selected ones.  With this library
    installed they run unchanged; checked here against the reference's torch backend with the same options.

    That host logic depends on the ORDER in which the top-k operator returns a row (it keeps "the first k - 20 non-special
    candidates", it pads an expanded list by repeating its head), and the reference asks its own operators for unsorted
    lists (``torch.topk(sorted=False)``, ``indexer.py:602``; ``VGGT_INDEXER_TOPK_SORTED`` off), so two correct backends
    differ there by construction.  Both runs therefore get their lists in one canonical order (ascending index) at the
    caller's entry ``LightningIndexer.select_topk_projected``; what remains is the operators' work on the shapes these
    options produce.  With pooled keys the two backends also pool in different precisions (fp32 for the torch backend,
    ``geoweave/inference.py:56-58``), which moves a cell at the cut in some rows: those rows are counted, the others
    must agree."""
    import geoweave_b200

    rh.enable_import()
    topk = 512
    blk = rh.build_block("vggt", topk, seed=4, device=dev(), dtype=torch.bfloat16)
    x, pos = rh.make_inputs("vggt", VIEWS, seed=4, device=dev(), dtype=torch.bfloat16)
    N = x.shape[1]
    select = blk.attn.indexer.select_topk_projected

    def canonical(*a, **k):
        r = select(*a, **k)
        if isinstance(r, tuple):
            order = torch.argsort(r[0].long(), -1)
            return torch.gather(r[0], -1, order), (None if r[1] is None else torch.gather(r[1], -1, order))
        return torch.sort(r, -1).values

    monkeypatch.setattr(blk.attn.indexer, "select_topk_projected", canonical)
    got = {}
    hook = _proj_input_hook(blk, got)
    rh.set_backend(blk, "vggt", VIEWS, "torch", topk, **state)
    y_ref, cap_ref = rh.run_block(blk, "vggt", x, pos)
    o_ref = got.pop("o").float()
    rh.set_backend(blk, "vggt", VIEWS, "torch", topk)
    y_plain, _ = rh.run_block(blk, "vggt", x, pos)
    got.pop("o")
    assert (y_ref.float() - y_plain.float()).abs().max().item() > 0  # the option changes what is selected
    torch.cuda.empty_cache()
    geoweave_b200.install()
    try:
        calls = _Calls(monkeypatch)
        monkeypatch.setenv("VGGT_INDEXER_TOPK_INFER_DIRECT", "1")
        rh.set_backend(blk, "vggt", VIEWS, "kernel", topk, **state)
        y_ker, cap_ker = rh.run_block(blk, "vggt", x, pos)
        geoweave_b200.check_status()
    finally:
        hook.remove()
        geoweave_b200.uninstall()
    o_ker = got.pop("o").float()
    indexer_calls = calls.shapes.get("sparse_topk_indexer_inference_func", []) + calls.shapes.get("sparse_topk_indexer_func", [])
    attn_calls = sum(calls.n.get(n, 0) for n in ("sparse_index_flash_attn_func", "sparse_index_flash_attn_inference_func",
                                                 "sparse_index_flash_attn_inference_bhtd_func"))
    assert indexer_calls, calls.n
    if variant != "own_view_kept":  # there the caller masks a dense attention itself; only the selection is an operator call
        assert attn_calls == 1, calls.n
    pooled = variant.startswith("pooled")
    if variant == "pooled_sources":     # every query (in chunks) against the pooled keys
        assert sum(q[1] for q, _ in indexer_calls) == N and all(k[1] < N // 3 for _, k in indexer_calls), indexer_calls
    if variant == "pooled_queries_and_sources":
        assert all(q[1] < N // 3 and k[1] < N // 3 for q, k in indexer_calls), indexer_calls
    idx_ker, idx_ref = cap_ker.topk_indices.long(), cap_ref.topk_indices.long()
    assert tuple(idx_ker.shape) == tuple(idx_ref.shape) and int(idx_ker.min()) >= 0 and int(idx_ker.max()) < N
    same = (torch.sort(idx_ker, -1).values == torch.sort(idx_ref, -1).values).all(-1)[0]  # rows with the same multiset
    member = torch.zeros(N, N, dtype=torch.bool, device=dev())
    member.scatter_(1, idx_ref[0], True)
    overlap = member.gather(1, idx_ker[0]).float().mean().item()
    assert same.float().mean().item() >= (0.5 if pooled else 0.98), same.float().mean().item()
    assert overlap >= (0.99 if pooled else 0.999), overlap
    # outputs against the torch backend on the rows where both selected the same keys: attention, module, block
    assert (o_ker - o_ref)[0, same].abs().max().item() <= 2e-2
    assert (cap_ker.attn_out.float() - cap_ref.attn_out.float())[0, same].abs().max().item() <= 2e-2
    assert (y_ker.float() - y_ref.float())[0, same].abs().max().item() <= 2e-2


def test_reference_block_trains_through_this_library(monkeypatch):
    """The sparse TRAINING stage of the reference (``compute_loss``: the indexer's KL loss on the selected scores against
    the attention's ``attn_sum``, ``dsa_attention.py:5404-5412``) with this library's differentiable operators: one
    forward + backward of the reference's block in train mode with its torch backend, one with the kernel backend;
    loss, input gradient and every parameter gradient must agree.  The reference's optional Triton loss kernel is
    switched off in both runs so that both use its torch formulation."""
    import geoweave_b200
    import geoweave_b200.custom_flash_attn.sparse_index_flash_attn as attn_mod
    import geoweave_b200.custom_indexer.sparse_topk_indexer as idx_mod

    rh.enable_import()
    import easyvolcap.official_vggt.layers.dsa_attention as da

    monkeypatch.setattr(da, "sparse_indexer_kl_loss", None)
    topk = 512
    blk = rh.build_block("vggt", topk, seed=6, device=dev(), dtype=torch.bfloat16)
    x0, pos = rh.make_inputs("vggt", VIEWS, seed=6, device=dev(), dtype=torch.bfloat16)
    d_y = torch.randn(x0.shape, generator=torch.Generator().manual_seed(0)).to(dev())
    backward_calls = {"attention": 0, "indexer": 0}
    for name, mod, fn_name in (("attention", attn_mod, "sparse_attention_backward"), ("indexer", idx_mod, "indexer_topk_backward")):
        fn = getattr(mod, fn_name)

        def counted(*a, _fn=fn, _name=name, **k):
            backward_calls[_name] += 1
            return _fn(*a, **k)

        monkeypatch.setattr(mod, fn_name, counted)
    res = {}
    for backend in ("torch", "kernel"):
        if backend == "kernel":
            geoweave_b200.install()
        try:
            rh.set_backend(blk, "vggt", VIEWS, backend, topk, compute_loss=True, detach_input=True, loss_weight=1.0,
                           sparse_flash_disable_attn_sum=False)
            blk.train()
            blk.zero_grad(set_to_none=True)
            x = x0.clone().requires_grad_()
            y, loss = blk(x, pos=pos)
            ((y.float() * d_y).sum() * 1e-3 + loss.float()).backward()
            geoweave_b200.check_status()
        finally:
            if backend == "kernel":
                geoweave_b200.uninstall()
        res[backend] = (loss.item(), x.grad.float().clone(), {n: p.grad.float().clone() for n, p in blk.named_parameters() if p.grad is not None})
        if backend == "torch":
            assert backward_calls == {"attention": 0, "indexer": 0}
    assert backward_calls == {"attention": 1, "indexer": 1}, backward_calls
    (loss_t, dx_t, g_t), (loss_k, dx_k, g_k) = res["torch"], res["kernel"]
    assert abs(loss_t - loss_k) <= 2e-2 * max(1.0, abs(loss_t)), (loss_t, loss_k)
    assert (dx_t - dx_k).abs().max().item() <= 2e-2 * dx_t.abs().max().item()
    assert set(g_t) == set(g_k) and any(n.startswith("attn.indexer.") for n in g_t) and "attn.qkv.weight" in g_t
    for n in g_t:
        assert (g_t[n] - g_k[n]).abs().max().item() <= 3e-2 * g_t[n].abs().max().item() + 1e-6, n


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
