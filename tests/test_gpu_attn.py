"""GPU parity: sparse attention forward through the C ABI, against reference-generated fixtures and the oracle."""
import pytest
import torch

import geoweave_b200
from oracle import gw_oracle as orc
from tests.gpu_util import dev, t

pytestmark = pytest.mark.gpu

ATTN_CASES = ["attn_h4", "attn_h16", "attn_tnes", "attn_d128", "attn_d32"]
BF16_TOL = 2e-2   # max-abs, bf16 output
FP32_TOL = 1e-4   # max-abs, fp32 input/output


@pytest.mark.parametrize("name", ATTN_CASES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_forward_matches_reference_fixture(golden, name, dtype):
    import geoweave_b200
    from geoweave_b200.custom_flash_attn.sparse_index_flash_attn import sparse_attention_forward

    c = golden[name]
    q, k, v = t(c["q"], dtype), t(c["k"], dtype), t(c["v"], dtype)
    tol = FP32_TOL if dtype == torch.float32 else BF16_TOL
    for idx_key, out_key, sum_key in (("idx", "out", "attn_sum"), ("idx_pad", "out_pad", "attn_sum_pad")):
        if idx_key not in c:
            continue
        o, attn_sum, lse = sparse_attention_forward(q, k, v, t(c[idx_key]), float(c["scale"]), True, True, "bthd")
        geoweave_b200.check_status()
        assert o.dtype == dtype and o.shape == q.shape and o.is_contiguous()
        assert (o.float().cpu() - torch.from_numpy(c[out_key])).abs().max().item() <= tol
        assert (attn_sum.cpu() - torch.from_numpy(c[sum_key])).abs().max().item() <= (1e-4 if dtype == torch.float32 else 2e-2)
        _, lse_ref, _ = orc.sparse_attention(q.float().cpu(), k.float().cpu(), v.float().cpu(), c[idx_key], float(c["scale"]))
        torch.testing.assert_close(lse.cpu(), lse_ref, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("name", ["attn_h16", "attn_h4"])
def test_bhtd_layout_and_strided_views(golden, name):
    from geoweave_b200.custom_flash_attn import (sparse_index_flash_attn_inference_bhtd_func,
                                                 sparse_index_flash_attn_inference_func)

    c = golden[name]
    q, k, v = t(c["q"], torch.bfloat16), t(c["k"], torch.bfloat16), t(c["v"], torch.bfloat16)
    idx = t(c["idx"])
    o_ref, none = sparse_index_flash_attn_inference_func(q, k, v, idx, None, False, float(c["scale"]), False)
    assert none is None
    qb, kb, vb = [x.transpose(1, 2).contiguous() for x in (q, k, v)]
    o_b, _ = sparse_index_flash_attn_inference_bhtd_func(qb, kb, vb, idx, None, False, float(c["scale"]), False)
    assert o_b.shape == qb.shape
    # head-major input runs the scalar kernel, token-major the tensor-core one: equal up to output rounding
    assert (o_b.transpose(1, 2).float() - o_ref.float()).abs().max().item() <= BF16_TOL
    # q/k/v as views of one fused [B,N,3,H,D] projection buffer, the layout DSAAttention produces
    if q.shape[1] == k.shape[1]:
        fused = torch.stack([q, k, v], dim=2).contiguous()
        o_v, _ = sparse_index_flash_attn_inference_func(fused[:, :, 0], fused[:, :, 1], fused[:, :, 2], idx, None, False,
                                                        float(c["scale"]), False)
        assert torch.equal(o_v, o_ref)


def test_autograd_entry_returns_attn_sum_and_refuses_bias(golden):
    from geoweave_b200.custom_flash_attn import sparse_index_flash_attn_func

    c = golden["attn_h4"]
    q, k, v = t(c["q"], torch.bfloat16), t(c["k"], torch.bfloat16), t(c["v"], torch.bfloat16)
    o, attn_sum = sparse_index_flash_attn_func(q, k, v, t(c["idx"]), None, False, float(c["scale"]))
    assert attn_sum.dtype == torch.float32 and attn_sum.shape == c["attn_sum"].shape
    torch.testing.assert_close(attn_sum.sum(-1).cpu(), torch.full(attn_sum.shape[:2], float(q.shape[2])), rtol=0, atol=2e-2)
    o_g, _ = sparse_index_flash_attn_func(q.clone().requires_grad_(), k, v, t(c["idx"]), None, False, float(c["scale"]))
    assert o_g.requires_grad and torch.equal(o_g.detach(), o)  # the differentiable path runs the same forward kernel
    with pytest.raises(NotImplementedError):
        sparse_index_flash_attn_func(q.detach(), k, v, t(c["idx"]), torch.zeros(1, device=dev()))


def test_all_padding_row_and_out_of_range_indices():
    from geoweave_b200.custom_flash_attn.sparse_index_flash_attn import sparse_attention_forward

    g = torch.Generator().manual_seed(11)
    q = torch.randn(1, 3, 16, 64, generator=g)
    k = torch.randn(1, 50, 16, 64, generator=g)
    v = torch.randn(1, 50, 16, 64, generator=g)
    idx = torch.randint(0, 50, (1, 3, 37), generator=g).to(torch.int32)
    idx[0, 1] = -1
    idx[0, 2, ::2] = 50 + 7  # >= S is padding too
    o, asum, lse = sparse_attention_forward(q.to(dev()), k.to(dev()), v.to(dev()), idx.to(dev()), None, True, True)
    o_ref, lse_ref, asum_ref = orc.sparse_attention(q, k, v, idx)
    assert (o.cpu() - o_ref).abs().max().item() <= FP32_TOL
    assert torch.equal(o[0, 1].cpu(), torch.zeros(16, 64)) and bool(torch.isinf(lse[0, :, 1]).all())
    assert (asum.cpu() - asum_ref).abs().max().item() <= 1e-4


@pytest.mark.parametrize("T,S,K", [(300, 4164, 1024), (64, 33312, 1024), (33, 1041, 1041)])
def test_production_shape_bf16(T, S, K):
    """16 heads x 64, k = 1024 as in the VGGT/Pi3 presets; oracle on the same bf16-rounded inputs."""
    from geoweave_b200.custom_flash_attn import sparse_index_flash_attn_inference_func

    g = torch.Generator().manual_seed(T + S)
    q = torch.randn(1, T, 16, 64, generator=g).bfloat16()
    k = torch.randn(1, S, 16, 64, generator=g).bfloat16()
    v = torch.randn(1, S, 16, 64, generator=g).bfloat16()
    idx = torch.stack([torch.randperm(S, generator=g)[:K] for _ in range(T)]).view(1, T, K).to(torch.int32)
    o, _ = sparse_index_flash_attn_inference_func(q.to(dev()), k.to(dev()), v.to(dev()), idx.to(dev()), None, False, 0.125)
    o_ref, _, _ = orc.sparse_attention(q, k, v, idx, 0.125)
    assert (o.float().cpu() - o_ref).abs().max().item() <= BF16_TOL


@pytest.mark.parametrize("T,S,K,H", [
    (300, 4164, 1024, 16),    # logits of a query fit the kernel's buffer: attn_sum comes out of the forward kernel
    (200, 4164, 1000, 8),     # K not a multiple of the batch of 16, eight heads
    (150, 4164, 2048, 16),    # beyond the buffer: separate K-only pass
    (4000, 2082, 512, 16),    # every CTA walks several queries: the buffer is handed from query to query
])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_attn_sum_with_padding_at_production_shapes(T, S, K, H, dtype):
    from geoweave_b200.custom_flash_attn import sparse_index_flash_attn_func

    g = torch.Generator().manual_seed(T + S + K + H)
    q = torch.randn(1, T, H, 64, generator=g).to(dtype)
    k = torch.randn(1, S, H, 64, generator=g).to(dtype)
    v = torch.randn(1, S, H, 64, generator=g).to(dtype)
    idx = torch.stack([torch.randperm(S, generator=g)[:K] for _ in range(T)]).view(1, T, K).to(torch.int32)
    idx[0, 1::7, 5::3] = -1      # scattered padding
    idx[0, 2, :] = -1            # a row of nothing but padding
    idx[0, 3, 1:] = S + 3        # a single live key
    o, asum = sparse_index_flash_attn_func(q.to(dev()), k.to(dev()), v.to(dev()), idx.to(dev()), None, False, 0.125)
    o_ref, _, asum_ref = orc.sparse_attention(q, k, v, idx, 0.125)
    assert (o.float().cpu() - o_ref).abs().max().item() <= BF16_TOL
    assert asum.dtype == torch.float32 and asum.shape == (1, T, K)
    assert (asum.cpu() - asum_ref).abs().max().item() <= 2e-3
    assert torch.equal(asum[0, 2].cpu(), torch.zeros(K)) and abs(float(asum[0, 3, 0]) - H) <= 1e-3


def test_dense_index_entry_equals_plain_softmax_attention():
    """dense_index_flash_attn_func (reference :3121): every key listed for every query = ordinary attention."""
    from geoweave_b200.custom_flash_attn import dense_index_flash_attn_func

    g = torch.Generator().manual_seed(77)
    for dtype, tol, (T, S, Hh) in ((torch.bfloat16, 2e-2, (70, 333, 16)), (torch.float32, 1e-4, (33, 129, 4))):
        q = torch.randn(2, T, Hh, 64, generator=g).to(dtype)
        k = torch.randn(2, S, Hh, 64, generator=g).to(dtype)
        v = torch.randn(2, S, Hh, 64, generator=g).to(dtype)
        o, attn_sum = dense_index_flash_attn_func(q.to(dev()), k.to(dev()), v.to(dev()), None, False, 0.125)
        geoweave_b200.check_status()
        p = torch.softmax(torch.einsum("bthd,bshd->bhts", q.float(), k.float()) * 0.125, -1)
        ref = torch.einsum("bhts,bshd->bthd", p, v.float())
        assert o.shape == q.shape and o.dtype == dtype
        assert (o.float().cpu() - ref).abs().max().item() <= tol
        assert attn_sum.shape == (2, T, S) and (attn_sum.cpu() - p.sum(1)).abs().max().item() <= (4e-3 if dtype != torch.float32 else 1e-4)
