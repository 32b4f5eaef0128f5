"""Order-independent comparison of backend results with the CPU oracle.

Receive order is unspecified, so rows are matched by their (source rank, source token) identity and
expert-major slots only have to be a permutation inside their expert's range -- the same criteria as
the reference's helpers (nano_ep/testing/native_dispatch.py:10-76, native_combine.py:168-195).
"""

from __future__ import annotations

import torch

from .oracle import reference_dispatch, reference_plan


def _cpu(t):
    return None if t is None else t.detach().cpu()


def assert_dispatch_matches(result, case_xs, case_indices, case_weights, num_experts, rank, *, expand, alignment, zero_padding, weighted=True):
    """Check one rank's ``NativeDispatchResult`` (any backend) against the oracle."""
    world = len(case_xs)
    local_experts = num_experts // world
    topk = case_indices[0].shape[1]
    hidden = case_xs[0].shape[1]
    expected = reference_dispatch(case_xs, case_indices, num_experts, case_weights if weighted else None, do_expand=expand, alignment=alignment)[rank]
    lay = expected.layout
    handle = result.handle
    meta = _cpu(handle.layout.recv_metadata).long()
    assert handle.layout.recv_metadata.dtype == torch.int32
    assert meta.shape == (lay.recv_count, topk + 2), (meta.shape, lay.recv_count)
    assert handle.layout.recv_count == lay.recv_count
    assert handle.layout.expanded_capacity == lay.expanded_capacity
    torch.testing.assert_close(_cpu(handle.layout.expert_counts), lay.expert_counts)
    torch.testing.assert_close(_cpu(handle.layout.expert_offsets), lay.expert_offsets)
    src, tok = meta[:, 0], meta[:, 1]
    prefix = torch.bincount(lay.src_ranks, minlength=world).cumsum(0)
    torch.testing.assert_close(_cpu(handle.layout.recv_rank_prefix), prefix)
    # rows are grouped by source rank
    assert (src[1:] >= src[:-1]).all(), "receive rows must be grouped by source rank"
    keys = list(zip(src.tolist(), tok.tolist()))
    assert len(set(keys)) == len(keys), "duplicate receive rows"
    order = torch.tensor(sorted(range(len(keys)), key=keys.__getitem__), dtype=torch.int64)
    torch.testing.assert_close(src[order], lay.src_ranks)
    torch.testing.assert_close(tok[order], lay.src_tokens)
    # snapshot, send counts, destination map
    torch.testing.assert_close(_cpu(handle.topk_idx), case_indices[rank])
    plan = reference_plan(case_indices[rank], num_experts, world)
    torch.testing.assert_close(_cpu(handle.send_counts), plan.send_counts)
    dst = _cpu(handle.dst_slots)
    assert dst.shape == (case_indices[rank].shape[0], world)
    assert ((dst >= 0) == plan.token_in_rank).all()

    x = _cpu(result.x)
    rows = lay.expanded_capacity if expand else lay.recv_count
    assert x.shape == (rows, hidden) and x.dtype == case_xs[0].dtype
    w = _cpu(result.topk_weights)
    if not weighted:
        assert w is None
    if expand:
        assert result.topk_idx is None
        slots = meta[:, 2:][order]
        valid = lay.local_topk_idx >= 0
        assert (slots[~valid] == -1).all()
        for e, count in enumerate(lay.expert_counts.tolist()):
            start = int(lay.expert_offsets[e])
            got = slots[lay.local_topk_idx == e].sort().values
            torch.testing.assert_close(got, torch.arange(start, start + count))
        got_rows, want_rows = slots[valid], lay.expanded_slots[valid]
        assert torch.equal(x[got_rows].view(torch.int16), expected.x[want_rows].view(torch.int16))
        if weighted:
            assert w.shape == (rows,)
            assert torch.equal(w[got_rows].view(torch.int32), expected.topk_weights[want_rows].view(torch.int32))
        slot_map = _cpu(handle.slot_map).long()
        assert slot_map.shape == (rows,)
        pad = torch.ones(rows, dtype=torch.bool)
        pad[got_rows] = False
        assert (slot_map[pad] == -1).all()
        flat_rows = order[:, None].expand_as(slots)[valid]
        flat_k = torch.arange(topk)[None, :].expand_as(slots)[valid]
        torch.testing.assert_close(slot_map[got_rows], flat_rows * topk + flat_k)
        if zero_padding:
            assert (x[pad].view(torch.int16) == 0).all(), "padding rows must be zero"
            if weighted:
                assert (w[pad] == 0).all()
    else:
        local = meta[:, 2:]
        torch.testing.assert_close(local[order], lay.local_topk_idx)
        torch.testing.assert_close(_cpu(result.topk_idx), local)
        assert result.topk_idx.dtype == torch.int64
        assert torch.equal(x[order].view(torch.int16), expected.x.view(torch.int16))
        if weighted:
            assert w.shape == (rows, topk)
            assert torch.equal(w[order].view(torch.int32), expected.topk_weights.view(torch.int32))
        assert _cpu(handle.slot_map).numel() == 0
    return expected


def source_reference(values, indices, rank, num_experts, world, *, expand, allow_multiple_reduction, bias=None):
    """Bit-accurate expected ``combine`` output of source ``rank``.

    ``values[t][k]`` is the bf16 expert output of choice k of token t (a [T,K,H] tensor).  Models each
    rounding boundary: separate rows (expanded, single reduction) are summed at the source in
    ascending k; otherwise the rows of one destination rank are first summed in FP32 and rounded to
    bf16 (identity for a single row), then the per-rank rows are summed in ascending first-k.
    """
    local = num_experts // world
    idx = indices[rank]
    T, K = idx.shape
    H = values.shape[-1]
    out = torch.zeros((T, H), dtype=torch.float32)
    for t in range(T):
        ks = [k for k in range(K) if idx[t, k] >= 0]
        if expand and not allow_multiple_reduction:
            for k in ks:
                out[t] += values[t, k].float()
        else:
            groups: dict[int, list[int]] = {}
            for k in ks:
                groups.setdefault(int(idx[t, k]) // local, []).append(k)
            for first_k in sorted(g[0] for g in groups.values()):
                g = next(g for g in groups.values() if g[0] == first_k)
                part = torch.zeros(H, dtype=torch.float32)
                for k in g:
                    part += values[t, k].float()
                out[t] += part.to(values.dtype).float()
    if bias is not None:
        out += bias.float()
    return out.to(values.dtype)
