"""GPU parity of the indexer's backward (gradients of the selected scores with respect to q_idx, k_idx and w) against
torch autograd through a plain gather formulation of the same scores in fp32, directly and through the public autograd
entry ``sparse_topk_indexer_func``."""
import pytest
import torch

import geoweave_b200
from tests.gpu_util import dev

pytestmark = pytest.mark.gpu


def reference_scores(q, k, w, idx, scale):
    """q [B,T,H,D], k [B,S,H,D], w [B,S,H] fp32 (requires_grad); idx int64 [B,T,K], entries outside [0,S) are padding.
    score[t,j] = sum_h w[idx,h] * relu(scale * <q[t,h], k[idx,h]>) -- the reference's LightningIndexer._compute_scores
    (official_vggt/layers/indexer.py:330-420) restricted to the selected keys."""
    B, S = k.shape[0], k.shape[1]
    valid = (idx >= 0) & (idx < S)
    safe = torch.where(valid, idx, torch.zeros_like(idx))
    bidx = torch.arange(B, device=q.device).view(B, 1, 1)
    z = torch.einsum("bthd,btkhd->btkh", q, k[bidx, safe]) * scale
    sc = (w[bidx, safe] * torch.relu(z)).sum(-1)
    return torch.where(valid, sc, torch.zeros_like(sc))


def make(B, T, S, H, K, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, T, H, 64, generator=g).to(dtype)
    k = torch.randn(B, S, H, 64, generator=g).to(dtype)
    w = torch.randn(B, S, H, generator=g).to(dtype)
    grad = torch.randn(B, T, K, generator=g)
    return q, k, w, grad


def check(got, ref, tol=1e-2):
    for name, a, b in zip(("dq", "dk", "dw"), got, ref):
        assert a.shape == b.shape, name
        err = (a.float() - b).abs().max().item()
        assert err <= tol * max(1.0, b.abs().max().item()), (name, err, b.abs().max().item())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,T,S,H,K", [(1, 150, 400, 4, 96), (2, 90, 250, 2, 33), (1, 300, 100, 4, 50), (1, 40, 3000, 1, 7),
                                       (1, 130, 200, 3, 64)])
def test_backward_of_given_lists_matches_autograd(dtype, B, T, S, H, K):
    from geoweave_b200.custom_indexer.sparse_topk_indexer import indexer_topk_backward

    q, k, w, grad = make(B, T, S, H, K, dtype, seed=T + S + K)
    g = torch.Generator().manual_seed(1)
    idx = torch.stack([torch.stack([torch.randperm(S, generator=g)[:K] for _ in range(T)]) for _ in range(B)]).to(torch.int32)
    idx[:, ::3, -4:] = -1        # padded tails
    idx[:, 1::7, 0] = S + 5      # an out-of-range entry
    idx[0, T // 2] = -1          # a query with no key at all
    got = indexer_topk_backward(q.to(dev()), k.to(dev()), w.to(dev()), idx.to(dev()), grad.to(dev()), 0.125)
    geoweave_b200.check_status()
    qr, kr, wr = [x.float().to(dev()).requires_grad_() for x in (q, k, w)]
    (reference_scores(qr, kr, wr, idx.to(dev()).long(), 0.125) * grad.to(dev())).sum().backward()
    for x, ref in zip(got, (q, k, w)):
        assert x.dtype == dtype and x.shape == ref.shape
    check(got, (qr.grad, kr.grad, wr.grad))


def test_autograd_entry_selects_then_differentiates_and_is_reproducible():
    from geoweave_b200.custom_indexer import sparse_topk_indexer_func

    B, T, H, K = 1, 700, 4, 128
    q, k, w, grad = make(B, T, T, H, K, torch.bfloat16, seed=11)
    w = w.abs()
    runs = []
    for rep in range(2):
        qd, kd, wd = [x.to(dev()).requires_grad_() for x in (q, k, w)]
        idx, sc = sparse_topk_indexer_func(qd, kd, wd, None, K, 0.125, 0)
        assert idx.dtype == torch.int32 and not idx.requires_grad and sc.requires_grad
        (sc.float() * grad.to(dev())).sum().backward()
        runs.append((idx, sc.detach(), qd.grad, kd.grad, wd.grad))
    geoweave_b200.check_status()
    for a, b in zip(runs[0][2:], runs[1][2:]):
        assert torch.equal(a, b)  # fixed summation order: bit-identical from run to run
    idx, sc = runs[0][:2]
    qr, kr, wr = [x.float().to(dev()).requires_grad_() for x in (q, k, w)]
    sc_ref = reference_scores(qr, kr, wr, idx.long(), 0.125)
    assert (sc.float() - sc_ref).abs().max().item() <= 2e-2 * max(1.0, sc_ref.abs().max().item())
    (sc_ref * grad.to(dev())).sum().backward()
    check(runs[0][2:], (qr.grad, kr.grad, wr.grad))


def test_no_gradient_no_graph_and_refusals():
    from geoweave_b200.custom_indexer import sparse_topk_indexer_func
    from geoweave_b200.custom_indexer.sparse_topk_indexer import indexer_topk_backward

    q, k, w, grad = make(1, 64, 64, 4, 16, torch.bfloat16, seed=2)
    idx, sc = sparse_topk_indexer_func(q.to(dev()), k.to(dev()), w.to(dev()), None, 16, None, 0)
    assert not sc.requires_grad
    qd = q.to(dev()).requires_grad_()
    idx, sc = sparse_topk_indexer_func(qd, k.to(dev()), w.to(dev()), None, 16, None, 0)
    (idx.float().sum() * 0).backward() if idx.requires_grad else None  # indices never carry a gradient
    assert qd.grad is None
    with pytest.raises(NotImplementedError):
        indexer_topk_backward(q.float().to(dev()), k.float().to(dev()), w.float().to(dev()), idx, grad.to(dev()), None)
    with pytest.raises(ValueError):
        indexer_topk_backward(q.to(dev()), k.to(dev()), w.to(dev()), idx, grad[:, :, :3].to(dev()), None)
