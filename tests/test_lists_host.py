"""``group_by_key`` on CPU: the fixed order in which the backward kernels walk the (query, slot) pairs of a key."""
import torch

from geoweave_b200._lists import group_by_key


def test_pairs_grouped_by_key_in_query_slot_order():
    g = torch.Generator().manual_seed(0)
    B, T, K, S = 2, 13, 7, 11
    pos = torch.randint(-2, S + 2, (B, T, K), generator=g, dtype=torch.int32)   # some padding on both sides
    order, start = group_by_key(pos, S)
    assert order.dtype == torch.int32 and start.dtype == torch.int32
    assert tuple(order.shape) == (B, T * K) and tuple(start.shape) == (B, S + 1)
    for b in range(B):
        flat = pos[b].reshape(-1)
        assert sorted(order[b].tolist()) == list(range(T * K))                   # a permutation of all pairs
        for s in range(S):
            pairs = order[b, start[b, s]: start[b, s + 1]].tolist()
            assert pairs == [i for i in range(T * K) if int(flat[i]) == s]      # ascending (query, slot): stable
        tail = order[b, start[b, S]:].tolist()                                   # padding entries behind the last key
        assert tail == [i for i in range(T * K) if not 0 <= int(flat[i]) < S]


def test_empty_keys_have_empty_ranges():
    pos = torch.tensor([[[5, 5, 5]]], dtype=torch.int32)
    order, start = group_by_key(pos, 8)
    assert start[0].tolist() == [0, 0, 0, 0, 0, 0, 3, 3, 3] and order[0].tolist() == [0, 1, 2]
