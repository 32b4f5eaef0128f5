"""One rank of the multi-GPU public-API test (run under torch.distributed.run, one GPU per rank).

Covers what the reference's distributed tier covers through its public API (tests/distributed/worker.py,
dispatch_worker.py, arena_worker.py, bootstrap_worker.py): two buffer lifetimes, both layouts, all case
kinds, bit-exact combine against a source-side rounding model, async + previous_event with delayed
producers, cached replays with an interleaved foreign dispatch, back-to-back arena reuse, bootstrap
fault injection with identical aggregated errors, bounded-wait failure detection, misuse errors; a gated slow reader
whose staged rows must survive peers that run ahead (dispatch_barrier_worker.py:116-158, arena_worker.py:119-139),
results that outlive newer operations under a slow consumer stream (dispatch_worker.py:161-194), back-to-back
combines on the single return area, and a synchronous operation followed by a standalone barrier.
"""

import os
import sys
import time
from datetime import timedelta
from unittest import mock

import torch
import torch.distributed as dist

from nanoep_b200 import CudaBuffer, EPConfig
from nanoep_b200.parallel import cuda_buffer
from nanoep_b200.testing.cases import make_case
from nanoep_b200.testing.checks import assert_dispatch_matches, source_reference


def choice_values(case, seed=11):
    gen = torch.Generator().manual_seed(seed)
    return [torch.randn(idx.shape[0], case.num_topk, case.hidden, generator=gen).to(torch.bfloat16) for idx in case.indices]


def expert_outputs(values, got, expand):
    meta = got.handle.layout.recv_metadata.cpu().long()
    H = values[0].shape[-1]
    if expand:
        y = torch.full((got.handle.layout.expanded_capacity, H), float("nan"), dtype=torch.bfloat16)
        for r in range(meta.shape[0]):
            for k, slot in enumerate(meta[r, 2:].tolist()):
                if slot >= 0:
                    y[slot] = values[int(meta[r, 0])][int(meta[r, 1]), k]
        return y.cuda()
    y = torch.zeros((meta.shape[0], H), dtype=torch.bfloat16)
    for r in range(meta.shape[0]):
        acc = torch.zeros(H)
        for k, e in enumerate(meta[r, 2:].tolist()):
            if e >= 0:
                acc += values[int(meta[r, 0])][int(meta[r, 1]), k].float()
        y[r] = acc.to(torch.bfloat16)
    return y.cuda()


def check_round_trip(buf, case, rank, world, expand, alignment, multiple, *, async_op, delayed):
    values = choice_values(case)
    producer = torch.cuda.Stream()
    with torch.cuda.stream(producer):
        if delayed and rank % 2 == 0:
            torch.cuda._sleep(20_000_000)  # this rank's inputs become ready late
        x, idx, w = case.xs[rank].cuda(), case.indices[rank].cuda(), case.weights[rank].cuda()
        ready = torch.cuda.Event()
        ready.record()
    got = buf.dispatch(x, topk_idx=idx, weights=w, do_expand=expand, alignment=alignment, zero_padding=True,
                       previous_event=ready, async_op=async_op)
    idx.fill_(0)  # the handle must hold its own snapshot
    if async_op:
        assert got.event is not None
        got.event.current_stream_wait()
    else:
        assert got.event is None
    torch.cuda.current_stream().synchronize()
    assert_dispatch_matches(got, case.xs, case.indices, case.weights, case.num_experts, rank,
                            expand=expand, alignment=alignment, zero_padding=True)
    y = expert_outputs(values, got, expand)
    bias = torch.randn(case.indices[rank].shape[0], case.hidden, generator=torch.Generator().manual_seed(5 + rank)).to(torch.bfloat16)
    if delayed and rank % 2 == 1:
        torch.cuda._sleep(20_000_000)  # a slow consumer before combine
    back = buf.combine(y, got.handle, weights=got.topk_weights, bias=bias.cuda(), async_op=async_op)
    if async_op:
        back.event.current_stream_wait()
    torch.cuda.current_stream().synchronize()
    want = source_reference(values[rank], case.indices, rank, case.num_experts, world, expand=expand,
                            allow_multiple_reduction=multiple, bias=bias)
    assert torch.equal(back.x.cpu().view(torch.int16), want.view(torch.int16)), "combine is not bit-exact"
    want_w = case.weights[rank].masked_fill(case.indices[rank] < 0, 0)
    torch.testing.assert_close(back.topk_weights.cpu(), want_w, rtol=0, atol=0)
    return got


def lifetime(group, rank, world, multiple):
    checks = 0
    with CudaBuffer(group, EPConfig(3 * world, 3, 512, 2153), allow_multiple_reduction=multiple, wait_timeout_s=20.0) as buf:
        for kind in ("random", "empty", "masked", "skew", "mixed"):
            case = make_case(world, kind=kind, seed=17, hidden=512, tokens=37)
            for expand in (False, True):
                for async_op in (False, True):
                    got = check_round_trip(buf, case, rank, world, expand, 4 if expand else 1, multiple,
                                           async_op=async_op, delayed=(kind == "random"))
                    checks += 1
            # cached replay after an interleaved foreign (fresh) dispatch with other routing
            other = make_case(world, kind="mixed", seed=99, hidden=512, tokens=37)
            buf.dispatch(other.xs[rank].cuda(), topk_idx=other.indices[rank].cuda())
            x2 = (case.xs[rank].float() * -2).to(torch.bfloat16)
            xs2 = [(x.float() * -2).to(torch.bfloat16) for x in case.xs]
            again = buf.dispatch(x2.cuda(), handle=got.handle, weights=case.weights[rank].cuda(), zero_padding=True)
            torch.cuda.synchronize()
            assert again.handle is got.handle
            assert_dispatch_matches(again, xs2, case.indices, case.weights, case.num_experts, rank,
                                    expand=True, alignment=4, zero_padding=True)
            checks += 1
        # the same round trips with the single-launch kernels for small calls forced on, then switched off
        from nanoep_b200.utils.build import load_extension

        ext = load_extension()
        before = ext.fused_limits()
        try:
            for limit in (1 << 20, 0):
                ext.set_fused_limits(dispatch_tokens=limit, fresh_tokens=limit)
                for kind in ("random", "masked"):
                    case = make_case(world, kind=kind, seed=31, hidden=512, tokens=37)
                    for expand in (False, True):
                        alignment = 4 if expand else 1
                        got = check_round_trip(buf, case, rank, world, expand, alignment, multiple, async_op=False, delayed=(kind == "random"))
                        again = buf.dispatch(case.xs[rank].cuda(), handle=got.handle, weights=case.weights[rank].cuda(), zero_padding=True)
                        torch.cuda.synchronize()
                        assert_dispatch_matches(again, case.xs, case.indices, case.weights, case.num_experts, rank,
                                                expand=expand, alignment=alignment, zero_padding=True)
                        checks += 1
        finally:
            ext.set_fused_limits(*before)
        # back-to-back async operations reusing the window without host syncs in between
        case = make_case(world, kind="random", seed=23, hidden=512, tokens=64)
        x, idx, w = case.xs[rank].cuda(), case.indices[rank].cuda(), case.weights[rank].cuda()
        kept = []
        for it in range(6):
            got = buf.dispatch(x, topk_idx=idx, weights=w, do_expand=True, alignment=8, zero_padding=True, async_op=True)
            got.event.current_stream_wait()
            back = buf.combine(got.x, got.handle, async_op=True)
            back.event.current_stream_wait()
            kept.append(back.x)
            if it == 2:
                buf.barrier()  # standalone barriers share the epoch sequence
        torch.cuda.synchronize()
        buf.check_status()
        mult = (case.indices[rank] >= 0).sum(1, keepdim=True).float()
        want = (case.xs[rank].float() * mult).to(torch.bfloat16)
        for out in kept:
            torch.testing.assert_close(out.cpu().float(), want.float(), rtol=2e-2, atol=2e-2)
        # misuse
        for bad in (
            lambda: buf.dispatch(x.float(), topk_idx=idx),
            lambda: buf.dispatch(x),
            lambda: buf.dispatch(x, topk_idx=idx, handle=got.handle),
            lambda: buf.dispatch(x, handle=got.handle, alignment=3),
            lambda: buf.dispatch(x[:, :256].contiguous(), topk_idx=idx),
            lambda: buf.combine(got.x[:, :256].contiguous(), got.handle),
        ):
            try:
                bad()
            except (ValueError, RuntimeError, TypeError):
                continue
            raise AssertionError("misuse accepted")
        foreign_handle = got.handle
    for bad in (lambda: buf.dispatch(x, topk_idx=idx), lambda: buf.combine(got.x, foreign_handle)):
        try:
            bad()
        except RuntimeError as e:
            assert "closed" in str(e)
        else:
            raise AssertionError("use after close accepted")
    buf.close()  # idempotent
    return checks


def slow_reader_keeps_its_rows(group, rank, world):
    """Rank 0's pull of dispatch d1 is held behind a gate kernel (a slow reader) while every other rank finishes d1 and
    queues d2 and d3 (cached, so their hosts do not wait).  d3 reuses d1's staging copy, so it must not start before
    rank 0 has read it: the staged bytes stay unchanged while the reader is pending, rank 0's result is exact once the
    gate opens, and afterwards every signal slot holds the epoch of the last operation."""
    from nanoep_b200.utils.build import load_extension

    ext = load_extension()
    case = make_case(world, kind="random", seed=41, hidden=256, tokens=23)
    cfg = EPConfig(case.num_experts, case.num_topk, case.hidden, 64)
    with CudaBuffer(group, cfg, wait_timeout_s=30.0) as buf:
        x, idx, w = case.xs[rank].cuda(), case.indices[rank].cuda(), case.weights[rank].cuda()
        first = buf.dispatch(x, topk_idx=idx, weights=w, do_expand=True, alignment=4, zero_padding=True)  # d0, staging copy 0
        torch.cuda.synchronize()
        layout = buf.window.layout()
        rows_d1 = slice(layout["stage_rows_offset"] + layout["stage_rows_stride"],
                        layout["stage_rows_offset"] + layout["stage_rows_stride"] + x.shape[0] * layout["row_bytes"])
        gate = torch.zeros(2, dtype=torch.int32).pin_memory()
        xs1 = [(t.float() * 3).to(torch.bfloat16) for t in case.xs]
        xs_late = [(t.float() * -5).to(torch.bfloat16) for t in case.xs]
        x1, late = xs1[rank].cuda(), xs_late[rank].cuda()
        torch.cuda.synchronize()
        if rank == 0:
            ext.set_test_gate(gate, 20.0)
        try:
            d1 = buf.dispatch(x1, topk_idx=idx, weights=w, do_expand=True, alignment=4, zero_padding=True, async_op=True)
        finally:
            ext.set_test_gate(None)
        # d2 and d3 replay the routing with other payloads; d3 writes the staging copy that d1 used
        d2 = buf.dispatch(x, handle=first.handle, weights=w, zero_padding=True, async_op=True)
        d3 = buf.dispatch(late, handle=first.handle, weights=w, zero_padding=True, async_op=True)
        time.sleep(0.3)  # let the other ranks' GPUs run as far as they can
        # While the gate is shut nothing but plain copies is issued on this GPU: a kernel on any stream may be queued by
        # the hardware behind the kernels the gate holds back, and the host would then wait for the gate's own limit.
        staged = buf.window.local_window()[rows_d1].cpu()
        if rank == 0:
            assert not d1.event.query(), "the gated pull finished early"
        want = xs1[rank].view(torch.uint8).view(x.shape[0], -1)
        got_rows = staged.view(x.shape[0], layout["row_bytes"])[:, : 2 * case.hidden]
        assert torch.equal(got_rows, want), "staged rows changed while a reader was pending"
        dist.barrier(group=group)
        gate[0] = 1  # open the gate (only rank 0 ever waits on it); a host store, no GPU work that could queue behind it
        for pending in (d1, d2, d3):
            pending.event.current_stream_wait()
        torch.cuda.synchronize()
        assert int(gate[1]) == 0, "the gate ran into its own limit"
        buf.check_status()
        assert_dispatch_matches(d1, xs1, case.indices, case.weights, case.num_experts, rank, expand=True, alignment=4, zero_padding=True)
        assert_dispatch_matches(d3, xs_late, case.indices, case.weights, case.num_experts, rank, expand=True, alignment=4, zero_padding=True)
        signals = buf.window.local_window()[layout["signal_offset"] : layout["signal_offset"] + 8 * world].view(torch.int64).cpu()
        assert (signals == buf.window.last_epoch).all(), (signals.tolist(), buf.window.last_epoch)


def back_to_back_combines(group, rank, world, multiple):
    """Combines that follow one another without a dispatch in between share the single return area: a rank may only
    overwrite a peer's partitions once that peer has reduced the previous contents, however the ranks are skewed."""
    case = make_case(world, kind="random", seed=53, hidden=512, tokens=41)
    cfg = EPConfig(case.num_experts, case.num_topk, case.hidden, 64)
    with CudaBuffer(group, cfg, allow_multiple_reduction=multiple, wait_timeout_s=30.0) as buf:
        x, idx, w = case.xs[rank].cuda(), case.indices[rank].cuda(), case.weights[rank].cuda()
        got = buf.dispatch(x, topk_idx=idx, weights=w, do_expand=True, alignment=8, zero_padding=True)
        outs, wants = [], []
        for it in range(8):
            values = choice_values(case, seed=100 + it)
            y = expert_outputs(values, got, True)
            if (it + rank) % 2 == 0:
                torch.cuda._sleep(15_000_000)  # alternate which ranks run late
            outs.append(buf.combine(y, got.handle).x)
            wants.append(source_reference(values[rank], case.indices, rank, case.num_experts, world, expand=True,
                                          allow_multiple_reduction=multiple))
        torch.cuda.synchronize()
        buf.check_status()
        for it, (out, want) in enumerate(zip(outs, wants)):
            assert torch.equal(out.cpu().view(torch.int16), want.view(torch.int16)), f"combine {it} of a back-to-back series is wrong"


def traced_combine_reports_its_roles(group, rank, world):
    """With the in-kernel time stamps switched on a combine still returns the exact sums, and the stamps are
    consistent: transfers end before the last flag is out, every token is summed once, the roles end in order."""
    from nanoep_b200.utils.build import load_extension

    ext = load_extension()
    case = make_case(world, kind="random", seed=61, hidden=512, tokens=57)
    cfg = EPConfig(case.num_experts, case.num_topk, case.hidden, 64)
    with CudaBuffer(group, cfg, wait_timeout_s=30.0) as buf:
        x, idx, w = case.xs[rank].cuda(), case.indices[rank].cuda(), case.weights[rank].cuda()
        got = buf.dispatch(x, topk_idx=idx, weights=w, do_expand=True, alignment=8, zero_padding=True)
        values = choice_values(case, seed=7)
        y = expert_outputs(values, got, True)
        ext.set_combine_trace(True, 0, 0)
        try:
            out = buf.combine(y, got.handle).x
            torch.cuda.synchronize()
            stamps = ext.take_combine_trace()
        finally:
            ext.set_combine_trace(False, 0, 0)
        buf.check_status()
        want = source_reference(values[rank], case.indices, rank, case.num_experts, world, expand=True, allow_multiple_reduction=False)
        assert torch.equal(out.cpu().view(torch.int16), want.view(torch.int16)), "a traced combine returned different sums"
        assert len(stamps) == 9, stamps
        transfers, flags, reduced, waited, summing, tokens, longest, longest_at, last_seen = stamps
        assert 0 < transfers <= flags + 1e-3 and 0 < reduced, stamps
        assert tokens == case.xs[rank].shape[0], stamps
        assert 0 < longest <= summing + 1e-3 and last_seen <= reduced + 1e-3 and longest_at <= reduced + 1e-3, stamps
        assert waited >= 0, stamps


def results_outlive_newer_operations(group, rank, world):
    """A slow consumer stream still reads a dispatch result after the caller dropped it and newer dispatches allocated
    tensors of the same sizes on the communication stream: the completion event registered the result with the
    consumer stream, so the allocator must not hand its memory out again."""
    case = make_case(world, kind="random", seed=67, hidden=512, tokens=48)
    cfg = EPConfig(case.num_experts, case.num_topk, case.hidden, 64)
    with CudaBuffer(group, cfg, wait_timeout_s=30.0) as buf:
        x, idx, w = case.xs[rank].cuda(), case.indices[rank].cuda(), case.weights[rank].cuda()
        other = (case.xs[rank].float() * 7).to(torch.bfloat16).cuda()
        consumer = torch.cuda.Stream()
        got = buf.dispatch(x, topk_idx=idx, weights=w, do_expand=True, alignment=4, zero_padding=True, async_op=True)
        handle = got.handle
        with torch.cuda.stream(consumer):
            got.event.current_stream_wait()
            torch.cuda._sleep(60_000_000)  # the consumer gets to the result late
            late_copy = got.x.clone()
            late_weights = got.topk_weights.clone()
        del got  # the caller lets go of the result while the consumer stream has not read it yet
        newer = []
        for _ in range(4):
            newer.append(buf.dispatch(other, handle=handle, weights=w, zero_padding=True, async_op=True))
        for n in newer:
            n.event.current_stream_wait()
        torch.cuda.synchronize()
        buf.check_status()
        first = buf.dispatch(x, handle=handle, weights=w, zero_padding=True)  # what the first result must have been
        torch.cuda.synchronize()
        assert torch.equal(late_copy.view(torch.int16), first.x.view(torch.int16)), "a result was recycled under a slow consumer"
        assert torch.equal(late_weights, first.topk_weights)


def synchronous_operation_then_barrier(group, rank, world):
    """A synchronous cached dispatch queued behind a long kernel on the caller's stream, then a standalone barrier on the
    communication stream: the barrier must not overtake the dispatch (its epoch would release the peers early)."""
    case = make_case(world, kind="random", seed=71, hidden=256, tokens=29)
    cfg = EPConfig(case.num_experts, case.num_topk, case.hidden, 64)
    with CudaBuffer(group, cfg, wait_timeout_s=30.0) as buf:
        x, idx, w = case.xs[rank].cuda(), case.indices[rank].cuda(), case.weights[rank].cuda()
        got = buf.dispatch(x, topk_idx=idx, weights=w, do_expand=False)
        torch.cuda.synchronize()
        xs2 = [(t.float() * -2).to(torch.bfloat16) for t in case.xs]
        x2 = xs2[rank].cuda()
        for it in range(3):
            if rank % 2 == it % 2:
                torch.cuda._sleep(30_000_000)  # the caller's stream is busy when the dispatch is queued
            again = buf.dispatch(x2, handle=got.handle, weights=w)
            buf.barrier()
            torch.cuda.synchronize()
            buf.check_status()
            assert_dispatch_matches(again, xs2, case.indices, case.weights, case.num_experts, rank, expand=False, alignment=1, zero_padding=False)



def bootstrap_faults(group, rank, world):
    cfg = EPConfig(2 * world, 2, 256, 8)
    real_load = cuda_buffer._load_native

    def failing_load():
        if rank == 0:
            raise OSError("injected allocation failure")
        return real_load()

    with mock.patch.object(cuda_buffer, "_load_native", failing_load):
        try:
            CudaBuffer(group, cfg)
        except RuntimeError as e:
            message = str(e)
        else:
            raise AssertionError("allocation failure not reported")
    assert message == "CudaBuffer allocation/export failed: rank 0: OSError: injected allocation failure", message

    class FailingImport:
        def __init__(self, inner):
            self._inner = inner

        def __getattr__(self, name):
            return getattr(self._inner, name)

        def import_handles(self, handles, peer_devices=()):
            if rank == 0:
                raise RuntimeError("injected import failure")
            return self._inner.import_handles(handles, list(peer_devices))

    class PatchedBackend:
        def __init__(self, inner):
            self._inner = inner

        def __getattr__(self, name):
            return getattr(self._inner, name)

        def PeerWindow(self, *a):
            return FailingImport(self._inner.PeerWindow(*a))

    with mock.patch.object(cuda_buffer, "_load_native", lambda: PatchedBackend(real_load())):
        try:
            CudaBuffer(group, cfg)
        except RuntimeError as e:
            message = str(e)
        else:
            raise AssertionError("import failure not reported")
    assert message == "CudaBuffer import/stream failed: rank 0: RuntimeError: injected import failure", message
    # mismatched configuration is reported identically everywhere
    try:
        CudaBuffer(group, EPConfig(2 * world, 2, 256, 8 + rank))
    except ValueError as e:
        assert str(e) == "EPConfig mismatch across ranks"
    else:
        raise AssertionError("config mismatch accepted")
    # after the rollbacks a normal buffer still works
    with CudaBuffer(group, cfg) as buf:
        x = torch.ones(8, 256, dtype=torch.bfloat16, device="cuda")
        idx = torch.tensor([[2 * ((rank + 1) % world), 2 * ((rank + 1) % world) + 1]], device="cuda").repeat(8, 1)
        got = buf.dispatch(x, topk_idx=idx, do_expand=True)
        back = buf.combine(got.x, got.handle)
        torch.cuda.synchronize()
        assert (back.x == 2).all()


def missing_peer_is_detected(group, rank, world):
    """Rank `world-1` skips one collective: the others' bounded wait runs out and is reported on the
    host; no GPU faults, the context stays usable, close() still works."""
    cfg = EPConfig(2 * world, 2, 256, 8)
    buf = CudaBuffer(group, cfg, wait_timeout_s=0.5)
    try:
        if rank != world - 1:
            buf.barrier()
            torch.cuda.synchronize()
            try:
                buf.check_status()
            except RuntimeError as e:
                assert "barrier timed out" in str(e)
            else:
                raise AssertionError("missing peer not detected")
            assert torch.ones(3, device="cuda").sum().item() == 3
        dist.barrier(group=group)
    finally:
        buf.close()


def main():
    rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    torch.cuda.set_device(local)
    dist.init_process_group("gloo", timeout=timedelta(seconds=120))
    try:
        group = dist.group.WORLD
        checks = 0
        for multiple in (False, True):
            checks += lifetime(group, rank, world, multiple)
        bootstrap_faults(group, rank, world)
        if world > 1:
            slow_reader_keeps_its_rows(group, rank, world)
            results_outlive_newer_operations(group, rank, world)
            synchronous_operation_then_barrier(group, rank, world)
            traced_combine_reports_its_roles(group, rank, world)
            for multiple in (False, True):
                back_to_back_combines(group, rank, world, multiple)
            missing_peer_is_detected(group, rank, world)
        dist.barrier()
        print(f"NANOEP_RANK_OK={rank} checks={checks}", flush=True)
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())
