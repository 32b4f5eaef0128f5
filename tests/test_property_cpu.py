"""Property test (hypothesis): the vectorised receive planner of the CPU backend agrees with the
scalar-loop oracle for arbitrary routing, and a dispatch/combine round trip through per-rank layouts
conserves every token's contributions."""

import torch
from hypothesis import given, settings
from hypothesis import strategies as st

from nanoep_b200.parallel.cpu_buffer import receive_layout
from nanoep_b200.testing.oracle import reference_combine, reference_dispatch, reference_layout


@st.composite
def routing(draw):
    world = draw(st.sampled_from([1, 2, 4]))
    local = draw(st.integers(1, 4))
    experts = world * local
    topk = draw(st.integers(1, min(4, experts)))
    tables = []
    for _ in range(world):
        tokens = draw(st.integers(0, 6))
        rows = []
        for _ in range(tokens):
            chosen = draw(st.permutations(range(experts)))[:topk]
            mask = draw(st.lists(st.booleans(), min_size=topk, max_size=topk))
            rows.append([-1 if m else e for e, m in zip(chosen, mask)])
        tables.append(torch.tensor(rows, dtype=torch.int64).reshape(tokens, topk))
    alignment = draw(st.sampled_from([1, 2, 8]))
    return world, experts, tables, alignment


@settings(max_examples=60, deadline=None)
@given(routing())
def test_planner_matches_oracle(case):
    world, experts, tables, alignment = case
    local = experts // world
    for rank in range(world):
        want = reference_layout(tables, rank, experts, alignment)
        for expand in (False, True):
            meta, local_ids, slots, counts, offsets, prefix = receive_layout(tables, rank, local, alignment, expand)
            assert meta.shape[0] == want.recv_count
            torch.testing.assert_close(meta[:, 0].long(), want.src_ranks)
            torch.testing.assert_close(meta[:, 1].long(), want.src_tokens)
            torch.testing.assert_close(local_ids, want.local_topk_idx)
            torch.testing.assert_close(counts, want.expert_counts)
            torch.testing.assert_close(offsets, want.expert_offsets)
            torch.testing.assert_close(slots, want.expanded_slots)


@settings(max_examples=30, deadline=None)
@given(routing())
def test_round_trip_conserves_contributions(case):
    world, experts, tables, alignment = case
    xs = [torch.arange(t.shape[0] * 4, dtype=torch.float32).reshape(-1, 4) + 100 * r for r, t in enumerate(tables)]
    batches = reference_dispatch(xs, tables, experts, do_expand=True, alignment=alignment)
    out, _ = reference_combine([b.x for b in batches], batches, tables)
    for r in range(world):
        mult = (tables[r] >= 0).sum(1, keepdim=True).float()
        torch.testing.assert_close(out[r], xs[r] * mult)
