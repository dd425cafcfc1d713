"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch


def dev():
    return torch.device("cuda:0")


def t(x, dtype=None, device=None):
    out = torch.from_numpy(np.ascontiguousarray(x))
    if dtype is not None:
        out = out.to(dtype)
    return out.to(device or dev())


def sorted_idx(x):
    return torch.sort(x.to(torch.int64), dim=-1).values.cpu()


def make_indexer_inputs(T, S, Hi=4, Di=64, seed=0, dtype=torch.bfloat16, ties=False, negw=False, integer=False):
    g = torch.Generator().manual_seed(seed)
    if integer:
        q = torch.randint(-3, 4, (1, T, Hi, Di), generator=g).float()
        k = torch.randint(-3, 4, (1, S, Hi, Di), generator=g).float()
        w = torch.randint(0, 9, (1, S, Hi), generator=g).float() / 8.0
    else:
        q = torch.randn(1, T, Hi, Di, generator=g)
        k = torch.randn(1, S, Hi, Di, generator=g)
        w = torch.randn(1, S, Hi, generator=g) if negw else torch.rand(1, S, Hi, generator=g)
    if ties:  # duplicate 10 % of the key rows (k_idx AND w, otherwise no tie is produced)
        n_dup = max(1, S // 10)
        dst = torch.randperm(S, generator=g)[:n_dup]
        src = torch.randint(0, S, (n_dup,), generator=g)
        k[0, dst] = k[0, src]
        w[0, dst] = w[0, src]
    q, k, w = q.to(dtype), k.to(dtype), w.to(dtype)
    return q, k, w
