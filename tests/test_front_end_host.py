"""Host logic of the projection front-end (no GPU): parameter collection from a module shaped like the reference's
DSAAttention, the concatenation order the kernel relies on, and the refusal of CPU tensors."""
import types

import pytest
import torch

from oracle import gw_oracle as orc


def stand_in_attention(heads=2, idx_heads=4, dim=128, eps=1e-6, rope=True):
    g = torch.Generator().manual_seed(1)
    lin = lambda i, o: torch.nn.Linear(i, o)
    idx = types.SimpleNamespace(q_proj=lin(dim, idx_heads * 64), k_proj=lin(dim, idx_heads * 64), w_proj=lin(dim, idx_heads),
                                k_norm=torch.nn.LayerNorm(64), n_heads=idx_heads)
    attn = types.SimpleNamespace(qkv=lin(dim, 3 * heads * 64), q_norm=torch.nn.LayerNorm(64, eps=eps), k_norm=torch.nn.Identity(),
                                 rope=types.SimpleNamespace(base_frequency=100.0) if rope else None, num_heads=heads, indexer=idx)
    with torch.no_grad():
        for m in (attn.qkv, idx.q_proj, idx.k_proj, idx.w_proj, attn.q_norm, idx.k_norm):
            for prm in m.parameters():
                prm.copy_(torch.randn(prm.shape, generator=g))
    return attn


def test_params_follow_the_reference_concatenation_order():
    from geoweave_b200.front_end import params_from_module

    attn = stand_in_attention()
    prm = params_from_module(attn, max_position=12, dtype=torch.float32)
    assert prm.heads == 2 and prm.idx_heads == 4
    assert prm.weight.shape == (3 * 2 * 64 + 2 * 4 * 64 + 4, 128) and prm.bias.shape == (prm.weight.shape[0],)
    # rows: qkv, then the indexer's q_proj, k_proj, w_proj (dsa_attention.py:545-585)
    assert torch.equal(prm.weight[:384], attn.qkv.weight) and torch.equal(prm.weight[384:640], attn.indexer.q_proj.weight)
    assert torch.equal(prm.weight[640:896], attn.indexer.k_proj.weight) and torch.equal(prm.weight[896:], attn.indexer.w_proj.weight)
    assert prm.q_norm is not None and prm.q_norm[2] == pytest.approx(1e-6) and prm.k_norm is None  # Identity -> no LayerNorm
    assert prm.idx_k_norm is not None and prm.idx_k_norm[2] == pytest.approx(1e-5)
    assert prm.cos.shape == (12, 32) and prm.cos.dtype == torch.float32
    assert torch.equal(prm.cos[:, :16], prm.cos[:, 16:])  # cat(angles, angles)
    # the oracle on F.linear of these parameters agrees with the modules applied one by one
    x = torch.randn(1, 10, 128)
    pos = torch.randint(0, 12, (1, 10, 2))
    fused = torch.nn.functional.linear(x, prm.weight, prm.bias)
    q, k, v, qi, ki, w = orc.project_front_end(fused, pos, prm.cos, prm.sin, 2, 64, 4, 64, prm.q_norm, prm.k_norm, prm.idx_k_norm)
    qkv = attn.qkv(x).reshape(1, 10, 3, 2, 64)
    assert torch.allclose(v, qkv[:, :, 2], atol=1e-6) and torch.allclose(w, attn.indexer.w_proj(x), atol=1e-6)
    k_plain = orc._rope_2d(qkv[:, :, 1], pos, prm.cos, prm.sin)
    assert torch.allclose(k, k_plain, atol=1e-5)
    ki_ref = orc._rope_2d(attn.indexer.k_norm(attn.indexer.k_proj(x).view(1, 10, 4, 64)), pos, prm.cos, prm.sin)
    assert torch.allclose(ki, ki_ref, atol=1e-5)


def test_no_rope_module_means_no_tables():
    from geoweave_b200.front_end import params_from_module

    prm = params_from_module(stand_in_attention(rope=False), max_position=4, dtype=torch.bfloat16)
    assert prm.cos is None and prm.sin is None


def test_cpu_tensors_are_refused():
    from geoweave_b200.front_end import FrontEndParams, project_epilogue

    prm = FrontEndParams(torch.empty(0), None, 2, 4)
    with pytest.raises((ValueError, RuntimeError)):
        project_epilogue(torch.zeros(1, 3, 3 * 2 * 64 + 2 * 4 * 64 + 4), None, prm)
