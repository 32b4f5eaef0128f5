"""EPConfig validation and hand-checked oracle cases (CPU)."""

import pytest
import torch

from nanoep_b200 import EPConfig
from nanoep_b200.testing.cases import KINDS, balanced_routing, make_case, uniform_routing, zipf_routing
from nanoep_b200.testing.oracle import reference_combine, reference_dispatch, reference_layout, reference_plan


def test_config_validation():
    cfg = EPConfig(8, 2, 256, 16)
    assert cfg.local_experts(4) == 2
    with pytest.raises(ValueError):
        EPConfig(0, 1, 256, 1)
    with pytest.raises(ValueError):
        EPConfig(4, 5, 256, 1)
    with pytest.raises(ValueError):
        EPConfig(64, 33, 256, 1)
    with pytest.raises(TypeError):
        EPConfig(4.0, 1, 256, 1)
    with pytest.raises(ValueError):
        cfg.local_experts(3)
    with pytest.raises(Exception):
        cfg.hidden = 3  # frozen


def test_oracle_hand_case():
    # 2 ranks, 2 experts each, K=2.  rank0: t0 -> (0, 2), t1 -> (3, -1); rank1: t0 -> (1, 0)
    idx = [torch.tensor([[0, 2], [3, -1]]), torch.tensor([[1, 0]])]
    plan = reference_plan(idx[0], 4, 2)
    assert plan.send_counts.tolist() == [1, 2]
    assert plan.token_in_rank.tolist() == [[True, True], [False, True]]
    lay0 = reference_layout(idx, 0, 4, alignment=2)
    assert lay0.src_ranks.tolist() == [0, 1] and lay0.src_tokens.tolist() == [0, 0]
    assert lay0.local_topk_idx.tolist() == [[0, -1], [1, 0]]
    assert lay0.expert_counts.tolist() == [2, 1]
    assert lay0.expert_offsets.tolist() == [0, 2, 4]
    assert lay0.expanded_slots.tolist() == [[0, -1], [2, 1]]
    lay1 = reference_layout(idx, 1, 4)
    assert lay1.src_tokens.tolist() == [0, 1] and lay1.recv_count == 2 and lay1.expanded_capacity == 2
    xs = [torch.arange(8.0).reshape(2, 4), torch.arange(8.0, 12.0).reshape(1, 4)]
    ws = [torch.tensor([[0.5, 0.25], [1.0, 9.0]]), torch.tensor([[0.75, 0.125]])]
    got = reference_dispatch(xs, idx, 4, ws, do_expand=True, alignment=2)
    assert got[0].x[0].tolist() == xs[0][0].tolist() and got[0].x[2].tolist() == xs[1][0].tolist()
    assert got[0].x[3].abs().sum() == 0  # padding
    assert got[0].topk_weights.tolist() == [0.5, 0.125, 0.75, 0.0]
    # identity experts scaled by gate weight: combine returns sum_k w_k * x
    outs = [(b.x * b.topk_weights[:, None]) for b in got]
    res, w_back = reference_combine(outs, got, idx, [b.topk_weights for b in got])
    torch.testing.assert_close(res[0][0], xs[0][0] * 0.75)
    torch.testing.assert_close(res[0][1], xs[0][1] * 1.0)
    torch.testing.assert_close(res[1][0], xs[1][0] * 0.875)
    assert w_back[0].tolist() == [[0.5, 0.25], [1.0, 0.0]]


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("world", [1, 2, 4])
def test_oracle_round_trip_identity(kind, world):
    case = make_case(world, kind=kind, dtype=torch.float32, hidden=8)
    for expand in (False, True):
        batches = reference_dispatch(case.xs, case.indices, case.num_experts, case.weights, do_expand=expand, alignment=4)
        if expand:
            outs = [b.x for b in batches]
        else:
            outs = [b.x * (b.layout.local_topk_idx >= 0).sum(1, keepdim=True) for b in batches]
        res, _ = reference_combine(outs, batches, case.indices)
        for r in range(world):
            mult = (case.indices[r] >= 0).sum(1, keepdim=True).float()
            torch.testing.assert_close(res[r], case.xs[r] * mult)


def test_routing_generators():
    idx, w = balanced_routing(64, 32, 4, seed=1)
    assert idx.shape == (64, 4) and torch.allclose(w.sum(-1), torch.ones(64))
    assert all(len(set(r)) == 4 for r in idx.tolist())
    idx, w = zipf_routing(256, 64, 6, seed=2)
    frac = (idx < 0).float().mean().item()
    assert 0.03 < frac < 0.2
    for row in idx.tolist():
        kept = [e for e in row if e >= 0]
        assert len(set(kept)) == len(kept)
    idx, _ = uniform_routing(16, 8, 8, seed=3)
    assert sorted(idx[0].tolist()) == list(range(8))
