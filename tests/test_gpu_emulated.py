"""Dispatch/combine kernels on ONE GPU with a logical group (all ranks in one launch).

Numerics are compared with the CPU oracle (plain PyTorch fp32) and are exact: dispatch moves bits,
combine has a defined rounding order.
"""

import pytest
import torch

from nanoep_b200 import EmulatedGroup, EPConfig
from nanoep_b200.testing.cases import KINDS, make_case, zipf_routing
from nanoep_b200.testing.checks import assert_dispatch_matches, source_reference

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["split_launches", "single_launch"])
def launch_path(request):
    """Run a test once with the small-call single-launch kernels switched off and once with them forced on."""
    from nanoep_b200.utils.build import load_extension

    ext = load_extension()
    before = ext.fused_limits()
    if request.param == "single_launch":
        ext.set_fused_limits(dispatch_tokens=1 << 20, fresh_tokens=1 << 20)
    else:
        ext.set_fused_limits(dispatch_tokens=0, fresh_tokens=0)
    yield request.param
    ext.set_fused_limits(*before)


@pytest.fixture(params=["reduce_default", "reduce_in_registers", "reduce_ring_small_chunks"])
def reduce_path(request):
    """Run a test with each form of the combine's source-side sum: the default (two-stage shared-memory ring), the
    register path with two warps per token, and a four-stage ring with 128-byte chunks (many chunks per token)."""
    from nanoep_b200.utils.build import load_extension

    ext = load_extension()
    setting = {"reduce_default": 0, "reduce_in_registers": 2, "reduce_ring_small_chunks": -4001}[request.param]
    ext.set_combine_trace(False, 0, setting)
    yield request.param
    ext.set_combine_trace(False, 0, 0)


def _to_cuda(ts):
    return [t.cuda() for t in ts]


def _choice_values(case, seed=11):
    gen = torch.Generator().manual_seed(seed)
    return [torch.randn(idx.shape[0], case.num_topk, case.hidden, generator=gen).to(torch.bfloat16) for idx in case.indices]


def _expert_outputs(values, got, expand):
    meta = got.handle.layout.recv_metadata.cpu().long()
    H = values[0].shape[-1]
    if expand:
        y = torch.full((got.handle.layout.expanded_capacity, H), float("nan"), dtype=torch.bfloat16)
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


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("kind", KINDS)
def test_dispatch_layouts(world, kind):
    case = make_case(world, kind=kind, seed=5, hidden=256, tokens=11)
    cfg = EPConfig(case.num_experts, case.num_topk, case.hidden, case.capacity)
    with EmulatedGroup(world, cfg) as group:
        for expand in (False, True):
            for alignment in (1, 4, 16) if expand else (1,):
                for weighted in (True, False):
                    got = group.dispatch(
                        _to_cuda(case.xs), topk_idx=_to_cuda(case.indices), weights=_to_cuda(case.weights) if weighted else None,
                        do_expand=expand, alignment=alignment, zero_padding=True, num_sms=3,
                    )
                    torch.cuda.synchronize()
                    group.check_status()
                    for r in range(world):
                        assert_dispatch_matches(
                            got[r], case.xs, case.indices, case.weights, case.num_experts, r,
                            expand=expand, alignment=alignment, zero_padding=True, weighted=weighted,
                        )


@pytest.mark.parametrize("world,multiple", [(2, False), (4, True)])
def test_combine_reduce_paths_bit_exact(world, multiple, reduce_path):
    """Every form of the source-side sum gives the oracle's bits (same order of FP32 additions, one rounding)."""
    for kind in ("mixed", "masked", "skew"):
        case = make_case(world, kind=kind, seed=21, hidden=768, tokens=37)
        cfg = EPConfig(case.num_experts, case.num_topk, case.hidden, case.capacity)
        values = _choice_values(case, seed=5)
        with EmulatedGroup(world, cfg, allow_multiple_reduction=multiple) as group:
            for expand in (False, True):
                got = group.dispatch(_to_cuda(case.xs), topk_idx=_to_cuda(case.indices), weights=_to_cuda(case.weights),
                                     do_expand=expand, alignment=4, zero_padding=False)
                torch.cuda.synchronize()
                ys = [_expert_outputs(values, got[r], expand).cuda() for r in range(world)]
                biases = [torch.randn(idx.shape[0], case.hidden).to(torch.bfloat16).cuda() for idx in case.indices]
                back = group.combine(ys, [g.handle for g in got], weights=[g.topk_weights for g in got], bias=biases)
                torch.cuda.synchronize()
                group.check_status()
                for r in range(world):
                    want = source_reference(values[r], case.indices, r, case.num_experts, world, expand=expand,
                                            allow_multiple_reduction=multiple, bias=biases[r].cpu())
                    assert torch.equal(back[r].x.cpu().view(torch.int16), want.view(torch.int16)), (reduce_path, kind, expand, r)
                    want_w = case.weights[r].masked_fill(case.indices[r] < 0, 0)
                    torch.testing.assert_close(back[r].topk_weights.cpu(), want_w, rtol=0, atol=0)


@pytest.mark.parametrize("world", [2, 4])
def test_edge_geometries_bit_exact(world):
    """One expert per rank, top-1, more choices than local experts, a rank without tokens, all-masked routing, an
    alignment larger than any expert's count: dispatch and combine against the oracle, both reduction modes."""
    for seed, (experts_per_rank, topk, tokens, hidden, kind) in enumerate([
        (1, 1, 5, 256, "random"), (1, 2, 9, 256, "mixed"), (2, 4, 17, 512, "random"), (5, 6, 33, 256, "skew"),
        (3, 1, 1, 256, "random"), (4, 8, 12, 256, "empty"), (2, 3, 6, 256, "masked"),
    ]):
        case = make_case(world, kind=kind, seed=40 + seed, hidden=hidden, tokens=tokens, experts_per_rank=experts_per_rank, topk=topk)
        cfg = EPConfig(case.num_experts, case.num_topk, case.hidden, case.capacity)
        values = _choice_values(case, seed=3)
        for multiple in (False, True):
            with EmulatedGroup(world, cfg, allow_multiple_reduction=multiple) as group:
                for expand, alignment in ((False, 1), (True, 1), (True, 16)):
                    got = group.dispatch(_to_cuda(case.xs), topk_idx=_to_cuda(case.indices), weights=_to_cuda(case.weights),
                                         do_expand=expand, alignment=alignment, zero_padding=True)
                    torch.cuda.synchronize()
                    for r in range(world):
                        assert_dispatch_matches(got[r], case.xs, case.indices, case.weights, case.num_experts, r,
                                                expand=expand, alignment=alignment, zero_padding=True)
                    ys = [_expert_outputs(values, got[r], expand).cuda() for r in range(world)]
                    back = group.combine(ys, [g.handle for g in got])
                    torch.cuda.synchronize()
                    group.check_status()
                    for r in range(world):
                        want = source_reference(values[r], case.indices, r, case.num_experts, world, expand=expand,
                                                allow_multiple_reduction=multiple)
                        assert torch.equal(back[r].x.cpu().view(torch.int16), want.view(torch.int16)), (seed, multiple, expand, alignment, r)


@pytest.mark.parametrize("world,multiple", [(1, False), (2, False), (2, True), (8, False), (8, True)])
def test_combine_modes_bit_exact(world, multiple, launch_path):
    for kind in ("mixed", "masked", "empty", "skew"):
        case = make_case(world, kind=kind, seed=9, hidden=512, tokens=9)
        cfg = EPConfig(case.num_experts, case.num_topk, case.hidden, case.capacity)
        values = _choice_values(case)
        with EmulatedGroup(world, cfg, allow_multiple_reduction=multiple) as group:
            for expand in (False, True):
                got = group.dispatch(_to_cuda(case.xs), topk_idx=_to_cuda(case.indices), weights=_to_cuda(case.weights),
                                     do_expand=expand, alignment=4, zero_padding=False)
                torch.cuda.synchronize()
                ys = [_expert_outputs(values, got[r], expand).cuda() for r in range(world)]
                biases = [torch.randn(idx.shape[0], case.hidden).to(torch.bfloat16).cuda() for idx in case.indices]
                for use_bias in (False, True):
                    back = group.combine(ys, [g.handle for g in got], weights=[g.topk_weights for g in got],
                                         bias=biases if use_bias else None)
                    torch.cuda.synchronize()
                    group.check_status()
                    for r in range(world):
                        want = source_reference(values[r], case.indices, r, case.num_experts, world, expand=expand,
                                                allow_multiple_reduction=multiple, bias=biases[r].cpu() if use_bias else None)
                        assert torch.equal(back[r].x.cpu().view(torch.int16), want.view(torch.int16)), (kind, expand, use_bias, r)
                        want_w = case.weights[r].masked_fill(case.indices[r] < 0, 0)
                        torch.testing.assert_close(back[r].topk_weights.cpu(), want_w, rtol=0, atol=0)


def test_cached_replay_and_poison(launch_path):
    world = 4
    case = make_case(world, kind="random", seed=21, hidden=256, tokens=13)
    cfg = EPConfig(case.num_experts, case.num_topk, case.hidden, case.capacity)
    with EmulatedGroup(world, cfg) as group:
        for expand in (False, True):
            first = group.dispatch(_to_cuda(case.xs), topk_idx=_to_cuda(case.indices), weights=_to_cuda(case.weights),
                                   do_expand=expand, alignment=8, zero_padding=True)
            torch.cuda.synchronize()
            keep_meta = [f.handle.layout.recv_metadata.clone() for f in first]
            keep_x = [f.x.clone() for f in first]
            # poison every window between calls: nothing stale may leak into later results
            for w in group.windows:
                view = w.local_window()
                lay = w.layout()
                view[lay["stage_rows_offset"]:lay["meta_scratch_offset"]].fill_(0xA5)
            xs2 = [(x.float() * -3).to(torch.bfloat16) for x in case.xs]
            for weighted in (False, True):
                again = group.dispatch(_to_cuda(xs2), handles=[f.handle for f in first],
                                       weights=_to_cuda(case.weights) if weighted else None, zero_padding=True)
                torch.cuda.synchronize()
                group.check_status()
                for r in range(world):
                    assert again[r].handle is first[r].handle
                    assert torch.equal(again[r].handle.layout.recv_metadata, keep_meta[r])
                    assert_dispatch_matches(again[r], xs2, case.indices, case.weights, case.num_experts, r,
                                            expand=expand, alignment=8, zero_padding=True, weighted=weighted)
                    assert torch.equal(first[r].x, keep_x[r]), "earlier outputs must own their storage"


def test_special_bit_patterns_survive_dispatch_and_combine(launch_path):
    """Dispatch moves bits (NaN payloads, infinities, negative zero, denormals and gate weights included);
    combine propagates non-finite values like a plain fp32 sum does."""
    world = 2
    case = make_case(world, kind="random", seed=3, hidden=256, tokens=12)
    patterns = torch.tensor([0x7FC1, 0xFFFF, 0x7F80, 0xFF80, 0x8000, 0x0001, 0x8001, 0x7F7F], dtype=torch.int32).to(torch.int16)
    xs = []
    for r, x in enumerate(case.xs):
        bits = x.clone().view(torch.int16)
        bits[:, r::7] = patterns[(torch.arange(bits[:, r::7].shape[1]) + r) % len(patterns)]
        xs.append(bits.view(torch.bfloat16))
    ws = [w.clone() for w in case.weights]
    ws[0].view(torch.int32)[0, 0] = 0x7FC00001  # a NaN with a payload among the gate weights
    cfg = EPConfig(case.num_experts, case.num_topk, case.hidden, case.capacity)
    with EmulatedGroup(world, cfg) as group:
        for expand in (False, True):
            first = group.dispatch(_to_cuda(xs), topk_idx=_to_cuda(case.indices), weights=_to_cuda(ws), do_expand=expand, alignment=4,
                                   zero_padding=True)
            again = group.dispatch(_to_cuda(xs), handles=[f.handle for f in first], weights=_to_cuda(ws), zero_padding=True)
            torch.cuda.synchronize()
            group.check_status()
            for got in (first, again):
                for r in range(world):
                    assert_dispatch_matches(got[r], xs, case.indices, ws, case.num_experts, r, expand=expand, alignment=4,
                                            zero_padding=True)
        # combine: identity experts; a token with an infinity or a NaN in a column keeps it (or turns NaN), like the reference sum
        back = group.combine([g.x for g in again], [f.handle for f in first])
        torch.cuda.synchronize()
        group.check_status()
        for r in range(world):
            acc = torch.zeros(xs[r].shape, dtype=torch.float32)
            for k in range(case.num_topk):  # fp32 sum over the valid choices in ascending k, one bf16 round
                acc = torch.where((case.indices[r][:, k] >= 0)[:, None], acc + xs[r].float(), acc)
            want = acc.to(torch.bfloat16)
            got = back[r].x.cpu()
            finite = torch.isfinite(want.float())
            assert torch.equal(torch.isnan(got.float()), torch.isnan(want.float()))
            assert torch.equal(got.float()[finite], want.float()[finite])
            inf = torch.isinf(want.float())
            assert torch.equal(got.float()[inf], want.float()[inf])


def test_many_rounds_large_hidden():
    """More rows than one grid round per warp, DeepSeek-V3 row size, 260 experts on one rank."""
    torch.manual_seed(0)
    T, H, K, E = 3 * 148 + 5, 7168, 8, 260
    cfg = EPConfig(E, K, H, T)
    idx, w = zipf_routing(T, E, K, seed=4)
    x = torch.randn(T, H).to(torch.bfloat16)
    with EmulatedGroup(1, cfg) as group:
        got = group.dispatch([x.cuda()], topk_idx=[idx.cuda()], weights=[w.cuda()], do_expand=True, alignment=128,
                             zero_padding=True, num_sms=8)[0]
        torch.cuda.synchronize()
        group.check_status()
        assert_dispatch_matches(got, [x], [idx], [w], E, 0, expand=True, alignment=128, zero_padding=True)
        y = (got.x.float() * got.topk_weights[:, None]).to(torch.bfloat16)
        back = group.combine([y], [got.handle], weights=[got.topk_weights])[0]
        torch.cuda.synchronize()
        group.check_status()
        want = torch.zeros(T, H)
        for k in range(K):
            valid = (idx[:, k] >= 0).float()[:, None]
            want += (x.float() * w[:, k, None]).to(torch.bfloat16).float() * valid
        torch.testing.assert_close(back.x.cpu().float(), want.to(torch.bfloat16).float(), rtol=0, atol=0)


def test_bad_expert_id_reports_status():
    cfg = EPConfig(4, 2, 256, 4)
    with EmulatedGroup(1, cfg) as group:
        x = torch.zeros(4, 256, dtype=torch.bfloat16, device="cuda")
        idx = torch.tensor([[0, 1], [2, 9], [3, -1], [1, 0]], device="cuda")
        group.dispatch([x], topk_idx=[idx])
        torch.cuda.synchronize()
        with pytest.raises(RuntimeError, match="expert id"):
            group.check_status()
        # the status is sticky until cleared; afterwards the group works again
        with pytest.raises(RuntimeError, match="expert id"):
            group.dispatch([x], topk_idx=[idx.clamp(max=3)])
        for w in group.windows:
            w.clear_status(group.comm_stream.cuda_stream)
        got = group.dispatch([x], topk_idx=[idx.clamp(max=3)])[0]
        torch.cuda.synchronize()
        group.check_status()
        assert got.handle.layout.recv_count == 4


def test_barrier_timeout_is_reported_not_fatal():
    """A peer that never signals makes the bounded wait run out; the context stays usable."""
    cfg = EPConfig(4, 2, 256, 4)
    group = EmulatedGroup(2, cfg, wait_timeout_s=0.2)
    try:
        # only rank 0 enters the barrier: its wait for rank 1 must give up after ~0.2 s
        group.windows[0].barrier(group.comm_stream.cuda_stream)
        torch.cuda.synchronize()
        with pytest.raises(RuntimeError, match="barrier timed out"):
            group.windows[0].check_status()
        # the device is still healthy
        assert torch.ones(4, device="cuda").sum().item() == 4
    finally:
        torch.cuda.synchronize()
        group.close()


@pytest.mark.parametrize("world,tokens", [(2, 70), (4, 200), (8, 33)])
def test_receive_rows_follow_source_and_token_order(world, tokens):
    """A fresh dispatch places its receive rows by (source rank, source token): chunk prefixes, no atomics.  The combine
    relies on it (rows of one source token then arrive from all expert ranks at about the same time)."""
    case = make_case(world, kind="random", seed=21, hidden=256, tokens=tokens)
    cfg = EPConfig(case.num_experts, case.num_topk, case.hidden, case.capacity)
    with EmulatedGroup(world, cfg) as group:
        for expand in (False, True):
            got = group.dispatch(_to_cuda(case.xs), topk_idx=_to_cuda(case.indices), do_expand=expand, alignment=4 if expand else 1)
            torch.cuda.synchronize()
            group.check_status()
            for r in range(world):
                meta = got[r].handle.layout.recv_metadata.cpu().long()
                key = meta[:, 0] * (tokens + 1) + meta[:, 1]
                assert (key[1:] > key[:-1]).all(), f"rank {r}: receive rows are not in (source, token) order"
