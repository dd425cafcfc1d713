"""GPU: randomised shapes, dtypes and score distributions for the three operators, checked against plain torch
expressions evaluated on the same device (fp32) -- a net for shape- and data-dependent defects that the fixed
cases do not reach.  Seeds are fixed; every failure prints the drawn configuration."""
import pytest
import torch

from tests.gpu_util import dev

pytestmark = pytest.mark.gpu


def _ri(g, lo, hi):
    return int(torch.randint(lo, hi + 1, (1,), generator=g))


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_indexer_selection_is_a_valid_top_k_of_torch_scores(seed):
    """No duplicate or out-of-range index, nothing selected that lies below the k-th torch score by more than the
    fp32 rounding bound of its own dot products, nothing left out that lies above it by more than that bound."""
    import geoweave_b200
    from geoweave_b200.custom_indexer import sparse_topk_indexer_inference_func as indexer

    g = torch.Generator().manual_seed(seed)
    for _ in range(30):
        T = _ri(g, 1, 400)
        S = [_ri(g, 64, 4000), _ri(g, 4096, 9000), _ri(g, 9000, 70000), _ri(g, 70000, 200000)][_ri(g, 0, 3)]
        k = [_ri(g, 1, 64), _ri(g, 64, 512), 1024, _ri(g, 512, 2048)][_ri(g, 0, 3)]
        Hi, kind = _ri(g, 1, 4), _ri(g, 0, 4)
        q = torch.randn(1, T, Hi, 64, generator=g)
        kk = torch.randn(1, S, Hi, 64, generator=g)
        w = torch.rand(1, S, Hi, generator=g)
        if kind == 1:    # heavy-tailed key norms
            kk = kk * torch.exp(torch.randn(1, S, 1, 1, generator=g))
        elif kind == 2:  # few distinct keys: massive ties
            kk = kk[:, torch.randint(0, max(1, S // 50), (S,), generator=g)]
            w = w[:, :1].expand(1, S, Hi).contiguous()
        elif kind == 3:  # negative weights
            w = torch.randn(1, S, Hi, generator=g)
        elif kind == 4:  # half the keys near zero
            kk[:, : S // 2] *= 0.01
        dt = torch.bfloat16 if _ri(g, 0, 1) else torch.float16
        qd, kd, wd = q.to(dt).to(dev()), kk.to(dt).to(dev()), w.to(dt).to(dev())
        idx, _ = indexer(qd, kd, wd, None, k, 0.125, return_scores=False)
        geoweave_b200.check_status()
        cfg = dict(T=T, S=S, k=k, Hi=Hi, kind=kind, dtype=str(dt))
        keff = min(k, S)
        wt = wd.float().permute(0, 2, 1).unsqueeze(1)
        sc = (torch.relu(torch.einsum("bthd,bshd->bths", qd.float(), kd.float()) * 0.125) * wt).sum(2)
        srt = torch.sort(idx.long(), -1).values
        assert idx.shape[-1] == keff and int(srt.min()) >= 0 and int(srt.max()) < S, cfg
        assert not bool((srt[..., 1:] == srt[..., :-1]).any()), cfg
        kth = torch.topk(sc, keff, dim=-1).values[..., -1:]
        sel = torch.zeros_like(sc, dtype=torch.bool).scatter_(-1, idx.long(), True)
        bound = 3e-5 * (torch.einsum("bthd,bshd->bths", qd.float().abs(), kd.float().abs()) * 0.125 * wt.abs()).sum(2) + 1e-30
        assert int((sel & (sc < kth - bound)).sum()) == 0 and int((~sel & (sc > kth + bound)).sum()) == 0, cfg


@pytest.mark.parametrize("seed", [4, 5])
def test_stand_alone_top_k_equals_a_stable_sort(seed):
    from geoweave_b200.custom_indexer.topk_exact_cuda import topk_exact_select

    g = torch.Generator().manual_seed(seed)
    for _ in range(40):
        rows = _ri(g, 1, 300)
        cols = [_ri(g, 1, 2000), _ri(g, 2000, 9000), _ri(g, 9000, 56000), _ri(g, 56000, 120000)][_ri(g, 0, 3)]
        k = min(cols, [_ri(g, 1, 50), _ri(g, 50, 600), 1024, _ri(g, 600, 4096)][_ri(g, 0, 3)])
        kind = _ri(g, 0, 3)
        x = torch.randn(1, rows, cols, generator=g)
        if kind == 1:
            x = torch.round(x * 4) / 4
        elif kind == 2:
            x = torch.exp(4 * x)
        elif kind == 3:
            x = torch.relu(x - 1.5)
        dt = [torch.float32, torch.float32, torch.bfloat16, torch.float16][_ri(g, 0, 3)]
        xd = x.to(dt).to(dev())
        vals, pos = topk_exact_select(xd, k=k)
        ref = torch.sort(torch.sort(xd.float(), dim=-1, descending=True, stable=True).indices[..., :k], -1).values
        cfg = dict(rows=rows, cols=cols, k=k, kind=kind, dtype=str(dt))
        assert torch.equal(torch.sort(pos, -1).values, ref), cfg
        assert torch.equal(vals, xd.gather(-1, pos)), cfg


@pytest.mark.parametrize("seed", [6, 7])
def test_attention_with_random_padding_matches_torch(seed):
    import geoweave_b200
    from geoweave_b200.custom_flash_attn.sparse_index_flash_attn import sparse_attention_forward

    g = torch.Generator().manual_seed(seed)
    for _ in range(40):
        T, S = _ri(g, 1, 500), _ri(g, 1, 6000)
        K = [_ri(g, 1, 40), _ri(g, 40, 600), 1024, _ri(g, 600, 1500)][_ri(g, 0, 3)]
        H = [16, 8, 16, 4][_ri(g, 0, 3)]
        dt = [torch.bfloat16, torch.float16, torch.float32][_ri(g, 0, 2)]
        q = torch.randn(1, T, H, 64, generator=g).to(dt).to(dev())
        kk = torch.randn(1, S, H, 64, generator=g).to(dt).to(dev())
        v = torch.randn(1, S, H, 64, generator=g).to(dt).to(dev())
        pos = torch.randint(-S // 4 - 1, S + S // 4 + 1, (1, T, K), generator=g).to(torch.int32).to(dev())  # a third is padding
        want_sum = bool(_ri(g, 0, 1))
        o, asum, _ = sparse_attention_forward(q, kk, v, pos, None, want_sum, True, "bthd")
        geoweave_b200.check_status()
        valid = (pos >= 0) & (pos < S)
        safe = torch.where(valid, pos, torch.zeros_like(pos)).long()
        s = torch.einsum("thd,tkhd->thk", q.float()[0], kk.float()[0][safe[0]]) * 0.125
        pr = torch.nan_to_num(torch.softmax(s.masked_fill(~valid[0].unsqueeze(1), float("-inf")), -1), nan=0.0)
        ref = torch.einsum("thk,tkhd->thd", pr, v.float()[0][safe[0]])
        cfg = dict(T=T, S=S, K=K, H=H, dtype=str(dt), attn_sum=want_sum)
        assert bool(torch.isfinite(o.float()).all()), cfg
        assert (o.float()[0] - ref).abs().max().item() <= (1e-4 if dt == torch.float32 else 2e-2), cfg
        if want_sum:
            assert (asum[0] - pr.sum(1)).abs().max().item() <= (1e-4 if dt == torch.float32 else 4e-3), cfg


@pytest.mark.parametrize("seed", [11, 12])
def test_both_backward_passes_on_random_shapes_match_autograd(seed):
    """Random sizes, head counts, dtypes, padding and duplicates in the lists; with and without a gradient through
    attn_sum: the attention's dQ, dK, dV and the indexer's dq, dk, dw against torch autograd of plain formulations."""
    import geoweave_b200
    from geoweave_b200.custom_flash_attn import sparse_index_flash_attn_func
    from geoweave_b200.custom_indexer.sparse_topk_indexer import indexer_topk_backward

    g = torch.Generator().manual_seed(seed)
    for _ in range(12):
        T, S = _ri(g, 1, 300), _ri(g, 2, 2000)
        K = [_ri(g, 1, 20), _ri(g, 20, 200), _ri(g, 200, 400)][_ri(g, 0, 2)]
        H = [16, 8, 4, 2][_ri(g, 0, 3)]
        dt = [torch.bfloat16, torch.float16, torch.float32][_ri(g, 0, 2)]
        with_sum = bool(_ri(g, 0, 1))
        q, kk, v = [torch.randn(1, n, H, 64, generator=g).to(dt) for n in (T, S, S)]
        pos = torch.randint(-S // 5 - 1, S + S // 5 + 1, (1, T, K), generator=g).to(torch.int32)   # padding and duplicates
        d_o, d_a = torch.randn(1, T, H, 64, generator=g).to(dt), torch.randn(1, T, K, generator=g)
        cfg = dict(T=T, S=S, K=K, H=H, dtype=str(dt), with_sum=with_sum)
        qd, kd, vd = [x.to(dev()).requires_grad_() for x in (q, kk, v)]
        o, a = sparse_index_flash_attn_func(qd, kd, vd, pos.to(dev()), None, False, 0.125)
        loss = (o.float() * d_o.to(dev()).float()).sum() + ((a * d_a.to(dev())).sum() if with_sum else 0.0)
        loss.backward()
        geoweave_b200.check_status()
        qr, kr, vr = [x.float().to(dev()).requires_grad_() for x in (q, kk, v)]
        valid = ((pos >= 0) & (pos < S)).to(dev())
        safe = torch.where(valid, pos.to(dev()), torch.zeros_like(pos.to(dev()))).long()
        s = torch.einsum("thd,tkhd->thk", qr[0], kr[0][safe[0]]) * 0.125
        pr = torch.nan_to_num(torch.softmax(s.masked_fill(~valid[0].unsqueeze(1), float("-inf")), -1), nan=0.0)
        pr = torch.where(valid[0].unsqueeze(1), pr, torch.zeros_like(pr))
        o_ref = torch.einsum("thk,tkhd->thd", pr, vr[0][safe[0]])
        ((o_ref * d_o.to(dev()).float()[0]).sum() + ((pr.sum(1) * d_a.to(dev())[0]).sum() if with_sum else 0.0)).backward()
        tol = 2e-4 if dt == torch.float32 else 1e-2
        for name, got, ref in (("dq", qd.grad, qr.grad), ("dk", kd.grad, kr.grad), ("dv", vd.grad, vr.grad)):
            assert (got.float() - ref).abs().max().item() <= tol * max(1.0, ref.abs().max().item()), (name, cfg)
        if dt == torch.float32:
            continue  # the indexer's backward takes 16-bit operands
        Hi = _ri(g, 1, 4)
        qi, ki = [torch.randn(1, n, Hi, 64, generator=g).to(dt) for n in (T, S)]
        w = torch.randn(1, S, Hi, generator=g).to(dt)
        got = indexer_topk_backward(qi.to(dev()), ki.to(dev()), w.to(dev()), pos.to(dev()), d_a.to(dev()), 0.125)
        geoweave_b200.check_status()
        qr, kr, wr = [x.float().to(dev()).requires_grad_() for x in (qi, ki, w)]
        z = torch.einsum("thd,tkhd->tkh", qr[0], kr[0][safe[0]]) * 0.125
        sc = torch.where(valid[0], (wr[0][safe[0]] * torch.relu(z)).sum(-1), torch.zeros_like(z[..., 0]))
        (sc * d_a.to(dev())[0]).sum().backward()
        for name, a_, b_ in zip(("dq_idx", "dk_idx", "dw"), got, (qr.grad, kr.grad, wr.grad)):
            assert (a_.float() - b_).abs().max().item() <= 1e-2 * max(1.0, b_.abs().max().item()), (name, cfg, Hi)
