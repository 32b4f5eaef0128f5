"""Module-level rank functions for the Gloo (CPU) tests."""

import torch
import torch.distributed as dist

from nanoep_b200 import CpuBuffer, EPConfig
from nanoep_b200.testing.cases import make_case
from nanoep_b200.testing.checks import assert_dispatch_matches, source_reference


def round_trip_identity(rank, world):
    """Baseline config: 4 experts, top-2, H=256, 16 tokens; every token goes to both experts of the
    next rank with weight 0.5; identity experts scaled by the gate weight; combine(x) == x."""
    torch.manual_seed(0)
    cfg = EPConfig(num_experts=2 * world, num_topk=2, hidden=256, num_max_tokens_per_rank=16)
    x = torch.randn(16, 256).to(torch.bfloat16)
    dst = (rank + 1) % world
    idx = torch.tensor([[2 * dst, 2 * dst + 1]], dtype=torch.int64).repeat(16, 1)
    w = torch.full((16, 2), 0.5)
    with CpuBuffer(dist.group.WORLD, cfg) as buf:
        got = buf.dispatch(x, topk_idx=idx, weights=w, do_expand=True, zero_padding=True)
        y = (got.x.float() * got.topk_weights[:, None]).to(got.x.dtype)
        back = buf.combine(y, got.handle)
        torch.testing.assert_close(back.x, x)
        # compact layout too: one row per (token, rank) -> sum the weights locally
        got = buf.dispatch(x, topk_idx=idx, weights=w)
        scale = (got.topk_weights * (got.topk_idx >= 0)).sum(1, keepdim=True)
        back = buf.combine((got.x.float() * scale).to(got.x.dtype), got.handle, weights=got.topk_weights)
        torch.testing.assert_close(back.x, x)
        torch.testing.assert_close(back.topk_weights, w)
    return True


def all_kinds(rank, world, multiple):
    for kind in ("random", "empty", "masked", "skew", "mixed"):
        case = make_case(world, kind=kind, seed=3, hidden=64, tokens=7)
        cfg = EPConfig(case.num_experts, case.num_topk, case.hidden, case.capacity)
        with CpuBuffer(dist.group.WORLD, cfg, allow_multiple_reduction=multiple) as buf:
            for expand in (False, True):
                for alignment in (1, 4):
                    got = buf.dispatch(
                        case.xs[rank], topk_idx=case.indices[rank], weights=case.weights[rank],
                        do_expand=expand, alignment=alignment, zero_padding=True,
                    )
                    assert_dispatch_matches(
                        got, case.xs, case.indices, case.weights, case.num_experts, rank,
                        expand=expand, alignment=alignment, zero_padding=True,
                    )
                    # cached replay with new payload and without weights keeps the handle object
                    x2 = (case.xs[rank].float() * 2).to(torch.bfloat16)
                    again = buf.dispatch(x2, handle=got.handle)
                    assert again.handle is got.handle and again.topk_weights is None
                    # experts: value depends on (token, k) so misrouted rows are caught
                    T, K, H = case.indices[rank].shape[0], case.num_topk, case.hidden
                    values = _choice_values(case, world)
                    y = _expert_outputs(values, got, expand)
                    bias = torch.randn(T, H).to(torch.bfloat16)
                    back = buf.combine(y, got.handle, weights=got.topk_weights, bias=bias)
                    want = source_reference(values[rank], case.indices, rank, case.num_experts, world, expand=expand,
                                            allow_multiple_reduction=multiple, bias=bias)
                    assert torch.equal(back.x.view(torch.int16), want.view(torch.int16)), (kind, expand, alignment)
                    want_w = case.weights[rank].masked_fill(case.indices[rank] < 0, 0)
                    torch.testing.assert_close(back.topk_weights, want_w, rtol=0, atol=0)
    return True


def geometry_sweep(rank, world):
    """Edge geometries against the oracle: one expert per rank, top-1, more choices than local experts, a rank
    without tokens, both layouts, both reduction modes, alignment larger than any expert's count."""
    checked = 0
    for seed, (experts_per_rank, topk, tokens, hidden, kind) in enumerate([
        (1, 1, 5, 256, "random"), (1, 2, 9, 256, "mixed"), (2, 4, 17, 512, "random"), (5, 6, 33, 256, "skew"),
        (3, 1, 1, 256, "random"), (4, 8, 12, 256, "empty"), (2, 3, 6, 256, "masked"),
    ]):
        case = make_case(world, kind=kind, seed=40 + seed, hidden=hidden, tokens=tokens, experts_per_rank=experts_per_rank, topk=topk)
        cfg = EPConfig(case.num_experts, case.num_topk, case.hidden, case.capacity)
        for multiple in (False, True):
            with CpuBuffer(dist.group.WORLD, cfg, allow_multiple_reduction=multiple) as buf:
                for expand, alignment in ((False, 1), (True, 1), (True, 16)):
                    got = buf.dispatch(case.xs[rank], topk_idx=case.indices[rank], weights=case.weights[rank],
                                       do_expand=expand, alignment=alignment, zero_padding=True)
                    assert_dispatch_matches(got, case.xs, case.indices, case.weights, case.num_experts, rank,
                                            expand=expand, alignment=alignment, zero_padding=True)
                    values = _choice_values(case, world)
                    back = buf.combine(_expert_outputs(values, got, expand), got.handle)
                    want = source_reference(values[rank], case.indices, rank, case.num_experts, world, expand=expand,
                                            allow_multiple_reduction=multiple)
                    assert torch.equal(back.x.view(torch.int16), want.view(torch.int16)), (seed, multiple, expand, alignment)
                    assert back.topk_weights is None
                    checked += 1
    return checked


def special_bits(rank, world):
    """Dispatch moves bits: NaN payloads, infinities, negative zero and denormals arrive unchanged."""
    case = make_case(world, kind="random", seed=3, hidden=64, tokens=9)
    patterns = torch.tensor([0x7FC1, 0xFFFF, 0x7F80, 0xFF80, 0x8000, 0x0001, 0x8001, 0x7F7F], dtype=torch.int32).to(torch.int16)
    xs = []
    for r, x in enumerate(case.xs):
        bits = x.clone().view(torch.int16)
        bits[:, r::5] = patterns[(torch.arange(bits[:, r::5].shape[1]) + r) % len(patterns)]
        xs.append(bits.view(torch.bfloat16))
    ws = [w.clone() for w in case.weights]
    ws[0].view(torch.int32)[0, 0] = 0x7FC00001
    cfg = EPConfig(case.num_experts, case.num_topk, case.hidden, case.capacity)
    with CpuBuffer(dist.group.WORLD, cfg) as buf:
        for expand in (False, True):
            got = buf.dispatch(xs[rank], topk_idx=case.indices[rank], weights=ws[rank], do_expand=expand, alignment=4, zero_padding=True)
            assert_dispatch_matches(got, xs, case.indices, ws, case.num_experts, rank, expand=expand, alignment=4, zero_padding=True)
            again = buf.dispatch(xs[rank], handle=got.handle, weights=ws[rank], zero_padding=True)
            assert_dispatch_matches(again, xs, case.indices, ws, case.num_experts, rank, expand=expand, alignment=4, zero_padding=True)
    return True


def _choice_values(case, world):
    gen = torch.Generator().manual_seed(11)
    return [torch.randn(idx.shape[0], case.num_topk, case.hidden, generator=gen).to(torch.bfloat16) for idx in case.indices]


def _expert_outputs(values, got, expand):
    """Build the expert-output tensor a rank would produce from per-(source, token, k) values."""
    meta = got.handle.layout.recv_metadata.long()
    H = values[0].shape[-1]
    if expand:
        y = torch.zeros((got.handle.layout.expanded_capacity, H), dtype=torch.bfloat16)
        for r in range(meta.shape[0]):
            for k, slot in enumerate(meta[r, 2:].tolist()):
                if slot >= 0:
                    y[slot] = values[int(meta[r, 0])][int(meta[r, 1]), k]
        return y
    y = torch.zeros((meta.shape[0], H), dtype=torch.bfloat16)
    for r in range(meta.shape[0]):
        acc = torch.zeros(H)
        for k, e in enumerate(meta[r, 2:].tolist()):
            if e >= 0:
                acc += values[int(meta[r, 0])][int(meta[r, 1]), k].float()
        y[r] = acc.to(torch.bfloat16)
    return y


def misuse(rank, world):
    cfg = EPConfig(2 * world, 2, 64, 4)
    buf = CpuBuffer(dist.group.WORLD, cfg)
    other = CpuBuffer(dist.group.WORLD, cfg)
    x = torch.zeros(4, 64, dtype=torch.bfloat16)
    idx = torch.zeros(4, 2, dtype=torch.int64)
    idx[:, 1] = 1
    got = buf.dispatch(x, topk_idx=idx)
    for bad in (
        lambda: buf.dispatch(x),  # fresh needs routing
        lambda: buf.dispatch(x, topk_idx=idx, handle=got.handle),
        lambda: buf.dispatch(x, handle=got.handle, alignment=8),
        lambda: buf.dispatch(x, handle=got.handle, do_expand=True),
        lambda: other.dispatch(x, handle=got.handle),
        lambda: other.combine(got.x, got.handle),
        lambda: buf.dispatch(x, topk_idx=idx, alignment=0),
        lambda: buf.dispatch(x.float(), topk_idx=idx),
        lambda: buf.combine(got.x[:, :8], got.handle),
    ):
        try:
            bad()
        except (ValueError, RuntimeError):
            continue
        raise AssertionError("misuse was accepted")
    buf.close()
    buf.close()  # idempotent
    other.close()
    try:
        buf.dispatch(x, topk_idx=idx)
    except RuntimeError as e:
        assert "closed" in str(e)
    else:
        raise AssertionError("dispatch after close was accepted")
    return True


def mismatched_config(rank, world):
    cfg = EPConfig(2 * world, 2, 64, 4 + rank)
    try:
        CpuBuffer(dist.group.WORLD, cfg)
    except ValueError as e:
        return str(e)
    raise AssertionError("config mismatch not detected")
