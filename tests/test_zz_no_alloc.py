"""The allocation-free planning entry point must agree with the regular dispatch path.

Collected last on purpose (file name): a failure here cannot hide results of the other tests in a
run that stops at the first failure.  The entry point is called through its exported C symbol, twice
in a row, and compared with what ``EmulatedGroup.dispatch`` (the existing path, whose scratch lives
in the peer window) produces for the same routing.  Comparison is exact: the outputs are integers.
"""

import pytest
import torch

from nanoep_b200 import EmulatedGroup, EPConfig
from nanoep_b200.ops import noalloc
from nanoep_b200.testing.cases import zipf_routing

pytestmark = pytest.mark.gpu


def _sorted_rows(meta):
    meta = meta.cpu().long()
    order = torch.argsort(meta[:, 1], stable=True)
    return meta[order]


def _existing_metadata(world, cfg, xs, idxs, expand, alignment):
    with EmulatedGroup(world, cfg) as group:
        got = group.dispatch(xs, topk_idx=idxs, do_expand=expand, alignment=alignment)
        torch.cuda.synchronize()
        group.check_status()
        return [(g.handle.layout.recv_metadata.clone(), g.handle.layout.expert_offsets.clone(), g.handle.layout.expert_counts.clone()) for g in got]


def test_compact_rows_match_dispatch_two_calls():
    world, T, K, E, H = 2, 200, 4, 16, 256
    L = E // world
    cfg = EPConfig(E, K, H, T)
    lib = noalloc.library()  # exported C symbols
    assert hasattr(lib, "nep_plan_rows_noalloc")
    for call, seed in enumerate((3, 4)):  # two calls in a row share the cursor array
        idxs = [zipf_routing(T, E, K, seed=seed * 10 + r)[0].cuda() for r in range(world)]
        xs = [torch.zeros(T, H, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
        existing = _existing_metadata(world, cfg, xs, idxs, False, 1)
        for rank in range(world):
            meta_all = existing[rank][0].cpu().long()
            for src in range(world):
                want = _sorted_rows(meta_all[meta_all[:, 0] == src])
                topk32 = idxs[src].to(torch.int32).contiguous()
                meta_out = torch.full((T, K + 2), -7, dtype=torch.int32, device="cuda")
                count = torch.zeros(1, dtype=torch.int32, device="cuda")
                code = noalloc.plan_rows_noalloc(topk32, src, rank * L, L, None, False, meta_out, count)
                assert code == noalloc.OK, lib.nep_noalloc_last_error()
                torch.cuda.synchronize()
                n = int(count.item())
                assert n == want.shape[0], (call, rank, src)
                got = _sorted_rows(meta_out[:n])
                assert torch.equal(got, want), (call, rank, src)
                assert (meta_out[n:] == -7).all(), "rows beyond the count must stay untouched"


def test_expanded_slots_match_dispatch_two_calls():
    T, K, E, H, alignment = 333, 6, 40, 256, 8
    cfg = EPConfig(E, K, H, T)
    for seed in (11, 12):
        idx = zipf_routing(T, E, K, seed=seed)[0].cuda()
        x = torch.zeros(T, H, dtype=torch.bfloat16, device="cuda")
        meta, offsets, counts = _existing_metadata(1, cfg, [x], [idx], True, alignment)[0]
        want = _sorted_rows(meta)
        meta_out = torch.full((T, K + 2), -7, dtype=torch.int32, device="cuda")
        count = torch.zeros(1, dtype=torch.int32, device="cuda")
        code = noalloc.plan_rows_noalloc(idx.to(torch.int32).contiguous(), 0, 0, E, offsets.to(torch.int32).contiguous(), True, meta_out, count)
        assert code == noalloc.OK
        torch.cuda.synchronize()
        n = int(count.item())
        assert n == want.shape[0]
        got = _sorted_rows(meta_out[:n])
        assert torch.equal(got[:, :2], want[:, :2])
        # slot order inside an expert is unspecified: compare which expert each choice landed in and
        # that each expert's slots are exactly its range
        off = offsets.cpu()
        expert_of = lambda s: torch.where(s >= 0, torch.bucketize(s.clamp(min=0), off[1:], right=True), torch.full_like(s, -1))
        assert torch.equal(expert_of(got[:, 2:]), expert_of(want[:, 2:]))
        for e, c in enumerate(counts.cpu().tolist()):
            mine = got[:, 2:][expert_of(got[:, 2:]) == e].sort().values
            assert torch.equal(mine, torch.arange(int(off[e]), int(off[e]) + c))


def test_sizes_beyond_the_maximum_are_rejected():
    topk32 = torch.zeros(4, 2, dtype=torch.int32, device="cuda")
    meta_out = torch.zeros(4, 4, dtype=torch.int32, device="cuda")
    count = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert noalloc.plan_rows_noalloc(topk32, 0, 0, noalloc.MAX_LOCAL_EXPERTS + 1, None, False, meta_out, count) == noalloc.TOO_LARGE
    wide = torch.zeros(4, 33, dtype=torch.int32, device="cuda")
    assert noalloc.plan_rows_noalloc(wide, 0, 0, 8, None, False, meta_out, count) == noalloc.TOO_LARGE
    assert noalloc.plan_rows_noalloc(topk32, 0, 0, 8, None, True, meta_out, count) == noalloc.BAD_ARGUMENT


def test_empty_input_and_inconsistent_offsets():
    K, L = 2, 4
    meta_out = torch.full((8, K + 2), -7, dtype=torch.int32, device="cuda")
    count = torch.full((1,), 99, dtype=torch.int32, device="cuda")
    empty = torch.zeros(0, K, dtype=torch.int32, device="cuda")
    assert noalloc.plan_rows_noalloc(empty, 0, 0, L, None, False, meta_out, count) == noalloc.OK
    torch.cuda.synchronize()
    assert int(count.item()) == 0 and (meta_out == -7).all()
    # four tokens all choose expert 1, but the offsets leave it two slots: the count reports the misfit
    # and no slot outside expert 1's range is handed out
    topk32 = torch.tensor([[1, -1]] * 4, dtype=torch.int32, device="cuda")
    offsets = torch.tensor([0, 2, 4, 6, 8], dtype=torch.int32, device="cuda")
    assert noalloc.plan_rows_noalloc(topk32, 0, 0, L, offsets, True, meta_out, count) == noalloc.OK
    torch.cuda.synchronize()
    assert int(count.item()) == -1
    slots = meta_out[:4, 2].cpu()
    assert sorted(s for s in slots.tolist() if s >= 0) == [2, 3] and (slots == -1).sum() == 2
    # the next call starts from cleared cursors
    assert noalloc.plan_rows_noalloc(topk32[:2].contiguous(), 0, 0, L, offsets, True, meta_out, count) == noalloc.OK
    torch.cuda.synchronize()
    assert int(count.item()) == 2
