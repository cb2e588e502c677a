"""Routing / schedule oracle: invariants the reference's harness states."""
import numpy as np
import pytest

from oracle import routing


def test_topk_routing_matches_torch():
    import torch
    torch.manual_seed(0)
    logits = torch.randn(300, 16)
    vals, ids = torch.topk(logits, 4, dim=1)
    my_ids, my_w = routing.route_topk(logits.numpy(), 4)
    assert np.array_equal(my_ids, ids.numpy().astype(np.int32))
    np.testing.assert_allclose(my_w, torch.softmax(vals, dim=-1).numpy(), rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("world,tokens,topk,experts,padding", [(1, 512, 1, 4, 128), (1, 300, 2, 8, 256),
                                                               (2, 200, 4, 8, 128), (4, 64, 2, 16, 128)])
def test_schedule_invariants(world, tokens, topk, experts, padding):
    rng = np.random.default_rng(world * 1000 + tokens)
    routes = np.stack([np.stack([rng.permutation(experts)[:topk] for _ in range(tokens)]) for _ in range(world)])
    E = experts // world
    for rank in range(world):
        cap = (world * tokens * topk + E * (padding - 1) + 127) // 128 * 128
        s = routing.build_schedule(routes, rank * E, E, cap, padding)
        total = int(s["num_tokens"][0])
        assert total % padding == 0 and total <= cap
        assert np.array_equal(s["tokens_per_expert"],
                              np.bincount(routes.reshape(-1) - rank * E, minlength=experts)[:E] if rank == 0
                              else np.array([(routes == rank * E + e).sum() for e in range(E)]))
        off = s["expert_offsets"]
        for e in range(E):
            lo, n = off[e], s["tokens_per_expert"][e]
            seg_r, seg_t, seg_d = s["peer_rank"][lo:lo + n], s["peer_token_idx"][lo:lo + n], s["dest_row"][lo:lo + n]
            # every row really routes to e, and rows are ordered by (rank, token, slot)
            assert (routes[seg_r, seg_t, seg_d % topk] == rank * E + e).all()
            assert (seg_d // topk == seg_t).all()
            key = seg_r.astype(np.int64) * tokens * topk + seg_d
            assert (np.diff(key) > 0).all()
            assert (s["peer_rank"][lo + n:off[e + 1]] == -1).all()
            assert (s["block_expert"][lo // 128:off[e + 1] // 128] == e).all()
        assert (s["block_expert"][total // 128:] == -1).all()
        assert (s["peer_rank"][:total] >= 0).sum() == s["tokens_per_expert"].sum()


def test_concentrated_routing_leaves_empty_experts():
    routes = np.tile(np.arange(2, dtype=np.int32), (1, 100, 1))
    s = routing.build_schedule(routes, 0, 8, 1024, 128)
    assert list(s["tokens_per_expert"]) == [100, 100, 0, 0, 0, 0, 0, 0]
    assert int(s["num_tokens"][0]) == 256
    assert list(s["expert_offsets"]) == [0, 128, 256, 256, 256, 256, 256, 256, 256]


def test_capacity_overflow_is_an_error():
    routes = np.zeros((1, 300, 1), dtype=np.int32)
    with pytest.raises(ValueError):
        routing.build_schedule(routes, 0, 2, 256, 128)
