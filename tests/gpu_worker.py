"""One rank of the multi-GPU public-API test (run under torch.distributed.run, one GPU per rank).

Covers what the reference's distributed tier covers through its public API (tests/distributed/worker.py,
dispatch_worker.py, arena_worker.py, bootstrap_worker.py): two buffer lifetimes, both layouts, all case
kinds, bit-exact combine against a source-side rounding model, async + previous_event with delayed
producers, cached replays with an interleaved foreign dispatch, back-to-back arena reuse, bootstrap
fault injection with identical aggregated errors, bounded-wait failure detection, misuse errors.
"""

import os
import sys
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
                ext.set_fused_limits(dispatch_tokens=limit)
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
            missing_peer_is_detected(group, rank, world)
        dist.barrier()
        print(f"NANOEP_RANK_OK={rank} checks={checks}", flush=True)
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())
