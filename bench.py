"""Headline benchmark: expert-parallel dispatch + combine round trip.

Metric and configuration follow the reference's DeepSeek-V3-shape target: 4096 tokens per rank x hidden
7168 bf16, top-8 of 256 experts (contiguous placement), softmax top-k routing, expert-major layout
with zero padding, fresh dispatch followed by combine.  One process per GPU; weak scaling (tokens
per rank fixed).

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 20 --warmup 5

Rank 0 prints ONE JSON line.  ``value`` is the whole-job payload rate in GB/s: per step every rank
receives N deduplicated rows in dispatch and C_valid assignment rows come back in combine; bytes =
(sum over ranks of N + C_valid) * hidden * 2, divided by the slowest rank's device time per step.

Arms: ``--impl ours`` (default), ``--impl nccl`` (torch.distributed all_to_all_single + index ops, a
baseline), ``--impl reference`` (the reference package; not installable offline, prints why), ``--impl refkernels``
(context only: the reference's own code with its JIT replaced by ahead-of-time instantiations, built by
``python baseline/refkernels/build.py``; labelled as such in its JSON line).

After the timed steps the ``ours`` arm checks, untimed, what it has just timed: receive counts against a count
of the all-gathered routing, every dispatched row against its source token, and the round trip bit for bit.
The JSON line carries ``"verified"``; the process exits non-zero when the check fails.  It then runs the NCCL arm
on the same inputs in the same process and reports ``vs_baseline`` = NCCL ms per step / this arm's ms per step.
"""

from __future__ import annotations

import argparse
import contextlib
import gc
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from datetime import timedelta

REFERENCE_UNAVAILABLE = (
    "reference cannot be installed offline: its setup.py requires the DeepJIT submodule (third-party/deep_jit), "
    "which is empty in the mounted checkout, and its kernels are only reachable through that JIT"
)


def parse_args():
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", choices=("ours", "nccl", "reference", "refkernels"), default="ours")
    p.add_argument("--tokens", type=int, default=4096)
    p.add_argument("--hidden", type=int, default=7168)
    p.add_argument("--experts", type=int, default=256)
    p.add_argument("--topk", type=int, default=8)
    p.add_argument("--alignment", type=int, default=128)
    p.add_argument("--layout", choices=("expanded", "compact"), default="expanded")
    p.add_argument("--routing", choices=("balanced", "zipf", "uniform"), default="balanced")
    p.add_argument("--cached", action="store_true", help="reuse the routing handle after the first step")
    p.add_argument("--multiple-reduction", action="store_true")
    p.add_argument("--num-sms", type=int, default=None)
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--no-nccl-anchor", action="store_true", help="skip the NCCL arm that fills vs_baseline")
    p.add_argument("--detail", action="store_true", help="record per-kernel device times (median, max over ranks) in phases_us")
    p.add_argument("--trace", action="store_true",
                   help="after the timed steps, run a few more with the kernels' own %%globaltimer stamps switched on and report them per rank "
                        "in kernel_trace_us (combine: transfer warps done, flags published, reduce warps done, then the reduce groups' totals: "
                        "us waited, us summing, tokens, longest token, its start, last token's rows seen; stage: routing counted, rows "
                        "staged, peer barrier passed, tail done; microseconds from the kernel's first block)")
    return p.parse_args()


_SAMPLER_CHILD = r"""
import subprocess, sys, time
target, period = sys.argv[1], float(sys.argv[2])
sys.stdout = open(sys.argv[3], "a", buffering=1)
try:
    import pynvml as n
    n.nvmlInit()
    h = n.nvmlDeviceGetHandleByUUID(target if target.startswith("GPU-") else "GPU-" + target)
    reasons = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or n.nvmlDeviceGetCurrentClocksThrottleReasons
    bits = [("hw_slowdown", "nvmlClocksThrottleReasonHwSlowdown"), ("hw_thermal_slowdown", "nvmlClocksThrottleReasonHwThermalSlowdown"),
            ("sw_thermal_slowdown", "nvmlClocksThrottleReasonSwThermalSlowdown"), ("sw_power_cap", "nvmlClocksThrottleReasonSwPowerCap")]
    bits = [(name, int(getattr(n, attr))) for name, attr in bits if hasattr(n, attr)]
    print("source nvml", flush=True)
    while True:
        mask = int(reasons(h))
        active = ",".join(name for name, bit in bits if mask & bit) or "-"
        print(time.time(), n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM), n.nvmlDeviceGetMaxClockInfo(h, n.NVML_CLOCK_SM), active, flush=True)
        time.sleep(period)
except Exception:
    print("source nvidia-smi", flush=True)
    query = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
    while True:
        try:
            out = subprocess.run(["nvidia-smi", "--query-gpu=" + query, "--format=csv,noheader,nounits", "-i", target],
                                 capture_output=True, text=True, timeout=5).stdout.strip().splitlines()[0].split(",")
            active = ",".join(nm for nm, flag in zip(names, out[2:6]) if flag.strip().lower().startswith("active")) or "-"
            print(time.time(), float(out[0]), float(out[1]), active, flush=True)
        except Exception:
            pass
        time.sleep(max(period, 0.2))
"""


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU while the timed regions run.

    The sampling loop lives in a child process (NVML queries, read-only; ``nvidia-smi`` as fallback) so that
    it never competes with the benchmark's own thread for the interpreter, and it samples every 50 ms only:
    management-library queries and kernel launches on one GPU share driver locks; the parent only notes the
    wall-clock windows of its timed regions and keeps the samples that fall inside them.  Nothing is ever
    set or reset on the GPU.
    """

    def __init__(self, gpu_index: int, gpu_uuid: str | None = None, period_s: float = 0.05):
        self.windows: list[list[float]] = []
        self.source = None
        self.extended_s = 0.0
        target = gpu_uuid if gpu_uuid else str(gpu_index)
        fd, self._path = tempfile.mkstemp(prefix="nanoep_clocks_", suffix=".txt")
        os.close(fd)
        try:
            # samples go to a file, so that a long run can never block the child on a full pipe
            self._child = subprocess.Popen([sys.executable, "-c", _SAMPLER_CHILD, target, str(period_s), self._path],
                                           stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
        except OSError:
            self._child = None

    def wait_ready(self, limit_s: float = 20.0) -> bool:
        """Block (bounded) until the child has written its first sample, i.e. NVML is up."""
        deadline = time.time() + limit_s
        while self._child is not None and time.time() < deadline:
            try:
                with open(self._path) as f:
                    if sum(1 for _ in f) >= 2:
                        return True
            except OSError:
                pass
            if self._child.poll() is not None:
                return False
            time.sleep(0.01)
        return False

    def __enter__(self):
        self.windows.append([time.time(), float("inf")])
        return self

    def __exit__(self, *exc):
        self.windows[-1][1] = time.time()

    def summary(self) -> dict:
        lines = []
        if self._child is not None:
            self._child.terminate()  # this exact child only
            try:
                self._child.wait(timeout=10)
            except subprocess.TimeoutExpired:
                self._child.kill()
            self._child = None
        try:
            with open(self._path) as f:
                lines = f.read().splitlines()
            os.unlink(self._path)
        except OSError:
            pass
        sm, mx, reasons = [], [], set()
        for line in lines:
            parts = line.split()
            if parts[:1] == ["source"]:
                self.source = parts[1]
                continue
            try:
                ts, clock, top, active = float(parts[0]), float(parts[1]), float(parts[2]), parts[3]
            except (ValueError, IndexError):
                continue
            if any(lo <= ts <= hi for lo, hi in self.windows):
                sm.append(clock)
                mx.append(top)
                reasons.update(r for r in active.split(",") if r != "-")
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(mx) if mx else None,
            "reasons": sorted(reasons),
            "samples": len(sm),
            "source": self.source,
            "window": "timed regions" + (f" + {self.extended_s:.2f} s of the same steps repeated untimed right after them"
                                         if self.extended_s else ""),
        }


def merge_clock_summaries(per_rank: list[dict]) -> dict:
    """One record for the job from every rank's own GPU: the slowest median clock, the union of the reasons."""
    medians = [s["sm_mhz"] for s in per_rank if s["sm_mhz"] is not None]
    tops = [s["sm_max_mhz"] for s in per_rank if s["sm_max_mhz"] is not None]
    return {
        "sm_mhz": min(medians) if medians else None,
        "sm_max_mhz": max(tops) if tops else None,
        "reasons": sorted({r for s in per_rank for r in s["reasons"]}),
        "samples": sum(s["samples"] for s in per_rank),
        "source": per_rank[0]["source"],
        "window": per_rank[0]["window"],
        "per_rank_sm_mhz": [s["sm_mhz"] for s in per_rank],
    }


def gather_clock_summaries(summary: dict, world: int, control_group) -> dict:
    import torch.distributed as dist

    gathered = [None] * world
    dist.all_gather_object(gathered, summary, group=control_group)
    return merge_clock_summaries(gathered)


def make_inputs(args, rank, world, device):
    import torch

    from nanoep_b200.testing.cases import balanced_routing, uniform_routing, zipf_routing

    gen = torch.Generator().manual_seed(1234 + rank)
    x = torch.randn(args.tokens, args.hidden, generator=gen, dtype=torch.float32).to(torch.bfloat16)
    if args.routing == "balanced":
        idx, w = balanced_routing(args.tokens, args.experts, args.topk, seed=99 + rank)
    elif args.routing == "zipf":
        idx, w = zipf_routing(args.tokens, args.experts, args.topk, seed=99 + rank)
    else:
        idx, w = uniform_routing(args.tokens, args.experts, args.topk, seed=99 + rank)
    return x.pin_memory(), idx.pin_memory(), w.pin_memory()


def verify_round_trip(args, buf, rank, world, device, control_group, x, idx, w, expand):
    """One more dispatch + combine with identity experts, checked on the device.  Returns (ok, note)."""
    import torch
    import torch.distributed as dist

    E, K, H, T = args.experts, args.topk, args.hidden, args.tokens
    L = E // world
    lo = rank * L
    got = buf.dispatch(x, topk_idx=idx, weights=w, do_expand=expand, alignment=args.alignment, zero_padding=expand, num_sms=args.num_sms)
    back = buf.combine(got.x, got.handle, num_sms=args.num_sms)
    if device.type == "cuda":
        torch.cuda.synchronize()
    if hasattr(buf, "check_status"):
        buf.check_status()
    problems = []
    # every rank's tokens and routing (device tensors over NCCL on GPUs; the control group on a CPU backend)
    all_x = torch.empty((world, T, H), dtype=x.dtype, device=device)
    all_idx = torch.empty((world, T, K), dtype=idx.dtype, device=device)
    if world > 1:
        data_group = None if device.type == "cuda" else control_group
        dist.all_gather(list(all_x.unbind(0)), x, group=data_group)
        dist.all_gather(list(all_idx.unbind(0)), idx, group=data_group)
    else:
        all_x[0], all_idx[0] = x, idx
    mine = (all_idx >= lo) & (all_idx < lo + L)
    want_rows = int(mine.any(-1).sum().item())
    want_counts = torch.bincount((all_idx[mine] - lo).flatten(), minlength=L)
    layout = got.handle.layout
    if layout.recv_count != want_rows:
        problems.append(f"recv_count {layout.recv_count} != {want_rows}")
    if not torch.equal(layout.expert_counts.to(want_counts.dtype), want_counts):
        problems.append("expert_counts differ from a count of the gathered routing")
    meta = layout.recv_metadata.long()
    src_rows = all_x[meta[:, 0], meta[:, 1]] if meta.shape[0] else all_x.new_zeros((0, H))
    if expand:
        slots = meta[:, 2:]
        row_of, choice = torch.nonzero(slots >= 0, as_tuple=True)
        flat = slots[row_of, choice]
        if flat.numel() != int(want_counts.sum().item()) or flat.unique().numel() != flat.numel():
            problems.append("expert-major slots are not a one-to-one assignment")
        if not torch.equal(got.x[flat].view(torch.int16), src_rows[row_of].view(torch.int16)):
            problems.append("a dispatched row differs from its source token")
        used = torch.zeros(got.x.shape[0], dtype=torch.bool, device=device)
        used[flat] = True
        if bool((got.x[~used] != 0).any().item()):
            problems.append("padding rows are not zero")
        want_w = w[meta[row_of, 1]] if world == 1 else None  # gate weights are checked by the test suite at every size
        del want_w
    elif not torch.equal(got.x.view(torch.int16), src_rows.view(torch.int16)):
        problems.append("a dispatched row differs from its source token")
    # identity experts: the result is the token times the number of rows that came back for it, rounded once
    # (rows pre-reduced per rank are rounded once more per rank)
    valid = idx >= 0
    dest = torch.where(valid, idx // L, torch.full_like(idx, -1))
    per_rank = torch.stack([(dest == d).sum(-1) for d in range(world)], dim=-1).float()  # [T, R]
    xf = x.float()
    if expand and not args.multiple_reduction:
        want = (xf * per_rank.sum(-1, keepdim=True)).to(x.dtype)
    elif expand:
        want = sum((xf * per_rank[:, d : d + 1]).to(x.dtype).float() for d in range(world)).to(x.dtype)
    else:
        want = (xf * (per_rank > 0).sum(-1, keepdim=True).float()).to(x.dtype)
    if not torch.equal(back.x.view(torch.int16), want.view(torch.int16)):
        bad = int((back.x.view(torch.int16) != want.view(torch.int16)).any(-1).sum().item())
        problems.append(f"round trip differs from the expected sum in {bad} tokens")
    gathered = [None] * world
    dist.all_gather_object(gathered, problems, group=control_group)
    everything = [f"rank {r}: {p}" for r, ps in enumerate(gathered) for p in ps]
    note = "; ".join(everything) if everything else (
        "recv_count and expert_counts equal a host-independent count of the all-gathered routing; every dispatched row equals its source "
        "token bit for bit, padding rows are zero; combine(dispatch(x)) equals bf16(x * rows returned) bit for bit; checked on every rank")
    return not everything, note


def run_ours(args, rank, world, device, control_group):
    import torch
    import torch.distributed as dist

    from nanoep_b200 import CudaBuffer, EPConfig
    from nanoep_b200.utils.build import load_extension

    ext = load_extension()
    cfg = EPConfig(args.experts, args.topk, args.hidden, args.tokens)
    expand = args.layout == "expanded"
    hx, hidx, hw = make_inputs(args, rank, world, device)
    x, idx, w = hx.to(device), hidx.to(device), hw.to(device)
    # Inputs larger than L2: the timed steps rotate over several copies of the token matrix so that no
    # step finds its inputs cached (the outputs and window traffic of a step, ~1.5 GB, evict the rest).
    copies = max(2, -(-(192 << 20) // max(1, x.numel() * 2)))
    x_sets = [x] + [x.clone() for _ in range(copies - 1)]

    def sync_all():
        torch.cuda.synchronize()
        dist.barrier(group=control_group)

    def max_over_ranks(value: float) -> float:
        t = torch.tensor([value], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=control_group)
        return float(t.item())

    def sum_over_ranks(value: float) -> float:
        t = torch.tensor([value], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=control_group)
        return float(t.item())

    clocks = ClockSampler(device.index, str(torch.cuda.get_device_properties(device).uuid))  # child starts during warm-up
    with CudaBuffer(control_group, cfg, allow_multiple_reduction=args.multiple_reduction) as buf:
        state = {"handle": None}

        def step(xd, idxd, wd, previous_event=None):
            handle = state["handle"] if args.cached else None
            got = buf.dispatch(
                xd, topk_idx=None if handle is not None else idxd, weights=wd, handle=handle,
                do_expand=expand if handle is None else None, alignment=args.alignment if handle is None else None,
                zero_padding=expand, previous_event=previous_event, num_sms=args.num_sms,
            )
            if args.cached:
                state["handle"] = got.handle
            # identity experts: the received rows are returned as they are
            back = buf.combine(got.x, got.handle, num_sms=args.num_sms)
            return got, back

        for _ in range(args.warmup):
            got, back = step(x, idx, w)
        sync_all()
        buf.check_status()
        n_rows = got.handle.layout.recv_count
        c_valid = int(got.handle.layout.expert_counts.sum().item())
        c_padded = got.handle.layout.expanded_capacity
        combine_rows = c_valid if (expand and not args.multiple_reduction) else n_rows
        recv_from_remote = n_rows - int((got.handle.layout.recv_metadata[:, 0] == rank).sum().item())

        # ---- device-timed steps
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
        mids = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
        launches_before = ext.launch_count()
        if args.detail:
            ext.take_phase_timings()
            ext.set_phase_timing(True)
        clocks.wait_ready()
        # No cyclic-GC pauses inside the timed regions: a fresh dispatch has a host round trip per step, so a
        # pause on one rank is a wait in the peer barrier for all of them.  Switched back on at the end.
        gc.collect()
        gc.disable()
        sync_all()
        with clocks:
            wall0 = time.perf_counter()
            for i in range(args.steps):
                xi = x_sets[i % len(x_sets)]
                starts[i].record()
                handle = state["handle"] if args.cached else None
                got = buf.dispatch(
                    xi, topk_idx=None if handle is not None else idx, weights=w, handle=handle,
                    do_expand=expand if handle is None else None, alignment=args.alignment if handle is None else None,
                    zero_padding=expand, num_sms=args.num_sms,
                )
                mids[i].record()
                back = buf.combine(got.x, got.handle, num_sms=args.num_sms)
                ends[i].record()
            sync_all()
            wall = time.perf_counter() - wall0
        launches = ext.launch_count() - launches_before
        phases = None
        if args.detail:
            ext.set_phase_timing(False)
            by_name: dict[str, list[float]] = {}
            for name, us in ext.take_phase_timings():
                by_name.setdefault(name, []).append(us)
            phases = {name: max_over_ranks(statistics.median(v)) for name, v in by_name.items()}
        buf.check_status()
        step_ms = [s.elapsed_time(e) for s, e in zip(starts, ends)]
        disp_ms = [s.elapsed_time(m) for s, m in zip(starts, mids)]
        comb_ms = [m.elapsed_time(e) for m, e in zip(mids, ends)]
        total_ms = max_over_ranks(sum(step_ms))
        ms_per_step = total_ms / args.steps
        ordered = sorted(step_ms)
        step_percentiles = {
            name: max_over_ranks(ordered[min(len(ordered) - 1, int(q * len(ordered)))])
            for name, q in (("p10", 0.10), ("p50", 0.50), ("p90", 0.90))
        }
        disp_us = max_over_ranks(statistics.median(disp_ms)) * 1e3
        comb_us = max_over_ranks(statistics.median(comb_ms)) * 1e3
        bytes_per_step = sum_over_ranks(float(n_rows + combine_rows)) * args.hidden * 2
        nvlink_bytes = sum_over_ranks(float(recv_from_remote)) * args.hidden * 2  # dispatch direction only
        value = bytes_per_step / (ms_per_step * 1e-3) / 1e9

        # ---- correctness of what was just timed (untimed): the routing counts against a host count of the
        # gathered routing, every dispatched row against its source token, the round trip bit for bit
        verified, verify_note = verify_round_trip(args, buf, rank, world, device, control_group, x, idx, w, expand)

        kernel_trace = None
        if args.trace:
            knobs = (int(os.environ.get("NANOEP_COMBINE_STORE_DEPTH", 0)), int(os.environ.get("NANOEP_COMBINE_REDUCE_GROUP", 0)))
            ext.set_combine_trace(True, *knobs)
            seen = {"combine": [], "stage": []}
            for i in range(12):
                step(x_sets[i % len(x_sets)], idx, w)
                torch.cuda.synchronize()
                combine_stamps, stage_stamps = ext.take_combine_trace(), ext.take_stage_trace()
                if i >= 3:
                    seen["combine"].append(combine_stamps)
                    seen["stage"].append(stage_stamps)
                dist.barrier(group=control_group)
            ext.set_combine_trace(False, *knobs)
            mine = {k: [round(statistics.median(r[j] for r in rows), 1) for j in range(len(rows[0]))] if rows and rows[0] else []
                    for k, rows in seen.items()}
            gathered = [None] * world
            dist.all_gather_object(gathered, mine, group=control_group)
            kernel_trace = {k: [g[k] for g in gathered] for k in ("combine", "stage")}

        # ---- end to end through the public API: every step copies its inputs from pinned host memory (on a copy
        # stream, one step ahead) and reads its result back into pinned host memory (on a second copy stream,
        # overlapping the next step); the host touches each result once it is there.  Two passes: the headline reads
        # back a per-token metric of the result (the L2 norm of every combined token, one reduction kernel); the
        # second reads back the whole combined [T, H] tensor, which on a full node is bound by the host links.
        e2e = None
        if not args.no_e2e:
            up_stream, down_stream = torch.cuda.Stream(), torch.cuda.Stream()
            bufs = [(torch.empty_like(x), torch.empty_like(idx), torch.empty_like(w)) for _ in range(2)]
            h2d = hx.numel() * 2 + hidx.numel() * 8 + hw.numel() * 4

            def upload(slot):
                with torch.cuda.stream(up_stream):
                    for dst, src in zip(bufs[slot], (hx, hidx, hw)):
                        dst.copy_(src, non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record()
                return ev

            def end_to_end(whole_result: bool):
                shape = tuple(x.shape) if whole_result else (x.shape[0],)
                dtype = x.dtype if whole_result else torch.float32
                results_host = [torch.empty(shape, dtype=dtype).pin_memory() for _ in range(2)]
                elapsed = 0.0
                for phase, count in (("warm", 2), ("timed", args.steps)):
                    sync_all()
                    if phase == "timed":
                        clocks.__enter__()  # keep sampling clocks during the end-to-end timed region as well
                    t0 = time.perf_counter()
                    ready = upload(0)
                    landed = [None, None]
                    checksum = 0.0
                    for i in range(count):
                        slot = i & 1
                        nxt = upload(slot ^ 1) if i + 1 < count else None
                        xd, idxd, wd = bufs[slot]
                        # the comm stream waits for the copy through previous_event; the caller's stream too
                        torch.cuda.current_stream().wait_event(ready)
                        got, back = step(xd, idxd, wd, previous_event=ready)
                        result = back.x if whole_result else torch.linalg.vector_norm(back.x, dim=-1, dtype=torch.float32)
                        done = torch.cuda.Event()
                        done.record()
                        with torch.cuda.stream(down_stream):
                            down_stream.wait_event(done)
                            results_host[slot].copy_(result, non_blocking=True)
                            result.record_stream(down_stream)
                            landed[slot] = torch.cuda.Event()
                            landed[slot].record()
                        up_stream.wait_event(done)  # the next upload into this slot's inputs must not overtake this step
                        if i > 0:
                            landed[slot ^ 1].synchronize()
                            checksum += float(results_host[slot ^ 1].flatten()[0])  # the host reads the previous step's result
                        ready = nxt
                    landed[(count - 1) & 1].synchronize()
                    checksum += float(results_host[(count - 1) & 1].flatten()[0])
                    sync_all()
                    elapsed = time.perf_counter() - t0
                    if phase == "timed":
                        clocks.__exit__(None, None, None)
                return max_over_ranks(elapsed * 1e3) / args.steps, results_host[0].numel() * results_host[0].element_size()

            metric_ms, metric_bytes = end_to_end(whole_result=False)
            whole_ms, whole_bytes = end_to_end(whole_result=True)
            e2e = {
                "value": bytes_per_step / (metric_ms * 1e-3) / 1e9,
                "unit": "GB/s",
                "ms_per_step": metric_ms,
                "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": metric_bytes,
                "read_back": "per-token metric of every step's result (fp32 L2 norm of each combined token, [tokens] floats) into pinned host memory",
                "whole_result_read_back": {
                    "ms_per_step": whole_ms,
                    "value": bytes_per_step / (whole_ms * 1e-3) / 1e9,
                    "d2h_bytes_per_step": whole_bytes,
                    "note": "same loop reading the whole combined [tokens, hidden] bf16 tensor back every step; bound by the host links when every GPU of the node does it",
                },
            }
        timed_wall_s = (ms_per_step + (e2e["ms_per_step"] if e2e else 0.0)) * 1e-3 * args.steps  # same value on every rank
        if timed_wall_s < 0.5:
            # The timed regions are shorter than a few sampling periods: repeat the same device-timed
            # steps (not counted in any number) so that the clock record shows the GPU under this load.
            extra = max(args.steps, int(0.5 / max(ms_per_step * 1e-3, 1e-6)))
            sync_all()
            t0 = time.time()
            with clocks:
                for i in range(extra):
                    step(x_sets[i % len(x_sets)], idx, w)
                sync_all()
            clocks.extended_s = time.time() - t0
            buf.check_status()
        clock_summary = gather_clock_summaries(clocks.summary(), world, control_group)
        gc.enable()

    # ---- same-box anchor: the NCCL all_to_all_single arm on the same inputs, same steps, same process
    nccl = None
    if not args.no_nccl_anchor:
        try:
            nccl_line = run_nccl(args, rank, world, device, control_group, sample_clocks=False)
            nccl = {"ms_per_step": nccl_line["ms_per_step"], "dispatch_us": nccl_line["dispatch_us"], "combine_us": nccl_line["combine_us"]}
        except Exception as error:  # the anchor must never cost the headline number
            nccl = {"error": f"{type(error).__name__}: {error}"[:200]}

    line = {
        "metric": "ep_dispatch_combine_payload_GBps",
        "value": value,
        "unit": "GB/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": ms_per_step,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": (nccl["ms_per_step"] / ms_per_step) if nccl and "ms_per_step" in nccl else None,
        "vs_baseline_is": "this arm's steps per second / the NCCL all_to_all_single arm's, same inputs, same process, same box "
                          "(the reference publishes no number for this configuration and does not install offline)",
        "nccl_all_to_all": nccl,
        "verified": verified,
        "verify": verify_note,
        "dtype": "bf16",
        "data": "synthetic (seeded N(0,1) tokens, softmax top-k routing); no expert weights involved",
        "impl": "ours",
        "config": {
            "model": "DeepSeek-V3 MoE shape: hidden 7168, 256 experts, top-8" if (args.hidden, args.experts, args.topk) == (7168, 256, 8)
            else f"hidden {args.hidden}, {args.experts} experts, top-{args.topk}",
            "global_batch": args.tokens * world,
            "seq_len": args.tokens,
            "tokens_per_rank": args.tokens,
            "parallelism": f"ep{world}",
            "layout": args.layout,
            "alignment": args.alignment,
            "zero_padding": expand,
            "routing": args.routing,
            "cached_handle": args.cached,
            "allow_multiple_reduction": args.multiple_reduction,
            "l2": f"inputs larger than L2: timed steps rotate over {len(x_sets)} copies of the token matrix ({len(x_sets) * x.numel() * 2 >> 20} MiB > 126 MB); a step also writes ~1 GB of outputs/window",
            "value_formula": "(sum_ranks N_dedup_rows + combine_rows) * hidden * 2 B / max_rank device time",
            "value_uses": "mean: the sum of the timed steps' device times (max over ranks) / steps; step_ms_percentiles gives the spread",
            "host": "Python cyclic GC off inside the timed regions",
            "combine_knobs": {"NANOEP_COMBINE_REDUCE_GROUP": os.environ.get("NANOEP_COMBINE_REDUCE_GROUP", "default (-2000: two-stage shared-memory ring)"),
                              "NANOEP_COMBINE_STORE_DEPTH": os.environ.get("NANOEP_COMBINE_STORE_DEPTH", "default (2)")},
        },
        "dispatch_us": disp_us,
        "combine_us": comb_us,
        "step_ms_percentiles": step_percentiles,
        "rows": {"recv_dedup": n_rows, "assignments": c_valid, "padded_capacity": c_padded},
        "nvlink_dispatch_GBps_per_gpu": (nvlink_bytes / world) / (disp_us * 1e-6) / 1e9 if world > 1 else 0.0,
        "wall_ms_per_step": max_over_ranks(wall * 1e3) / args.steps,
        "gpu_launches": launches,
        "phases_us": phases,
        "kernel_trace_us": kernel_trace,
        "clocks": clock_summary,
        "e2e": e2e,
    }
    return line


def run_nccl(args, rank, world, device, control_group, sample_clocks=True):
    """Baseline: torch.distributed all_to_all_single over NCCL + index ops (sort, index_select, index_add)."""
    import torch
    import torch.distributed as dist

    hx, hidx, hw = make_inputs(args, rank, world, device)
    x, idx, w = hx.to(device), hidx.to(device), hw.to(device)
    E, K, H, T = args.experts, args.topk, args.hidden, args.tokens
    L = E // world
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    nccl = dist.group.WORLD

    def dispatch_combine():
        flat = idx.flatten()
        token_of = torch.arange(T, device=device).repeat_interleave(K)
        order = torch.argsort(flat, stable=True)  # expert-major send order
        send_rows = x[token_of[order]]  # [T*K, H]
        per_expert = torch.bincount(flat, minlength=E)
        send_counts = per_expert.view(world, L).sum(1)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=nccl)
        in_splits, out_splits = send_counts.tolist(), recv_counts.tolist()
        recv_expert_counts = torch.empty(world * L, dtype=per_expert.dtype, device=device)
        dist.all_to_all_single(recv_expert_counts, per_expert, group=nccl)
        recv = torch.empty(sum(out_splits), H, dtype=x.dtype, device=device)
        dist.all_to_all_single(recv, send_rows, out_splits, in_splits, group=nccl)
        # expert-major permutation on the receiver (source-major -> expert-major)
        expert_of = torch.repeat_interleave(torch.arange(L, device=device).repeat(world), recv_expert_counts)
        perm = torch.argsort(expert_of, stable=True)
        expert_in = recv[perm]
        mid = torch.cuda.Event(enable_timing=True)
        mid.record()
        # combine: inverse permutation, all_to_all back, weighted-free sum at the source
        back_rows = torch.empty_like(recv)
        back_rows[perm] = expert_in
        returned = torch.empty(T * K, H, dtype=x.dtype, device=device)
        dist.all_to_all_single(returned, back_rows, in_splits, out_splits, group=nccl)
        out = torch.zeros(T, H, dtype=torch.float32, device=device)
        out.index_add_(0, token_of[order], returned.float())
        return out.to(x.dtype), mid, recv.shape[0]

    clocks = ClockSampler(device.index, str(torch.cuda.get_device_properties(device).uuid)) if sample_clocks else contextlib.nullcontext()
    for _ in range(args.warmup):
        dispatch_combine()
    torch.cuda.synchronize()
    dist.barrier(group=control_group)
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    mids = []
    if sample_clocks:
        clocks.wait_ready()
    with clocks:
        for i in range(args.steps):
            flush.fill_(i & 0xFF)
            starts[i].record()
            _, mid, rows = dispatch_combine()
            ends[i].record()
            mids.append(mid)
        torch.cuda.synchronize()
        dist.barrier(group=control_group)
    t = torch.tensor([sum(s.elapsed_time(e) for s, e in zip(starts, ends))], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=control_group)
    ms_per_step = float(t.item()) / args.steps
    d = torch.tensor([statistics.median(s.elapsed_time(m) for s, m in zip(starts, mids))], dtype=torch.float64)
    dist.all_reduce(d, op=dist.ReduceOp.MAX, group=control_group)
    rows_t = torch.tensor([float(rows)], dtype=torch.float64)
    dist.all_reduce(rows_t, op=dist.ReduceOp.SUM, group=control_group)
    bytes_per_step = 2 * float(rows_t.item()) * H * 2
    if sample_clocks and ms_per_step * 1e-3 * args.steps < 0.5:
        # too short for a clock record: repeat the same steps untimed with the sampling window open (same count on every rank)
        t0 = time.time()
        with clocks:
            for _ in range(max(args.steps, int(0.5 / max(ms_per_step * 1e-3, 1e-6)))):
                dispatch_combine()
            torch.cuda.synchronize()
            dist.barrier(group=control_group)
        clocks.extended_s = time.time() - t0
    return {
        "metric": "ep_dispatch_combine_payload_GBps",
        "value": bytes_per_step / (ms_per_step * 1e-3) / 1e9,
        "unit": "GB/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": ms_per_step,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic",
        "impl": "nccl_all_to_all_single",
        "config": {
            "model": f"hidden {H}, {E} experts, top-{K}", "global_batch": T * world, "seq_len": T, "parallelism": f"ep{world}",
            "note": "one row per assignment (no per-rank dedup), expert-major permutation by index ops; bytes counted as rows moved each way",
        },
        "dispatch_us": float(d.item()) * 1e3,
        "combine_us": (ms_per_step - float(d.item())) * 1e3,
        "gpu_launches": 0,
        "clocks": gather_clock_summaries(clocks.summary(), world, control_group) if sample_clocks else None,
    }


def run_refkernels(args, rank, world, device, control_group):
    """Context only, NOT the reference arm: the reference's own Python package, host runtime and kernel templates,
    with its run-time JIT (which cannot be built offline) replaced by ahead-of-time instantiations
    (baseline/refkernels).  Same inputs, same timing and the same round-trip check as the ``ours`` arm."""
    import torch
    import torch.distributed as dist

    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "refkernels"))
    import build as refbuild

    nano_ep = refbuild.reference_package()
    cfg = nano_ep.EPConfig(args.experts, args.topk, args.hidden, args.tokens)
    hx, hidx, hw = make_inputs(args, rank, world, device)
    x, idx, w = hx.to(device), hidx.to(device), hw.to(device)
    copies = max(2, -(-(192 << 20) // max(1, x.numel() * 2)))
    x_sets = [x] + [x.clone() for _ in range(copies - 1)]

    def reduce_max(value):
        t = torch.tensor([value], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=control_group)
        return float(t.item())

    with nano_ep.CudaBuffer(control_group, cfg) as buf:
        def step(xd):
            got = buf.dispatch(xd, topk_idx=idx, weights=w, do_expand=True, alignment=args.alignment, zero_padding=True)
            return got, buf.combine(got.x, got.handle)

        for _ in range(args.warmup):
            got, back = step(x)
        torch.cuda.synchronize()
        dist.barrier(group=control_group)
        n_rows = got.handle.layout.recv_count
        c_valid = int(got.handle.layout.expert_counts.sum().item())
        starts, mids, ends = ([torch.cuda.Event(enable_timing=True) for _ in range(args.steps)] for _ in range(3))
        gc.collect()
        gc.disable()
        for i in range(args.steps):
            xi = x_sets[i % len(x_sets)]
            starts[i].record()
            got = buf.dispatch(xi, topk_idx=idx, weights=w, do_expand=True, alignment=args.alignment, zero_padding=True)
            mids[i].record()
            back = buf.combine(got.x, got.handle)
            ends[i].record()
        torch.cuda.synchronize()
        dist.barrier(group=control_group)
        gc.enable()
        step_ms = [a.elapsed_time(b) for a, b in zip(starts, ends)]
        ms_per_step = reduce_max(sum(step_ms)) / args.steps
        disp_us = reduce_max(statistics.median(a.elapsed_time(b) for a, b in zip(starts, mids))) * 1e3
        comb_us = reduce_max(statistics.median(a.elapsed_time(b) for a, b in zip(mids, ends))) * 1e3
        # the same identity-expert check as the ours arm: token times the number of rows that came back, rounded once
        got, back = step(x)
        torch.cuda.synchronize()
        count = (idx >= 0).sum(-1, keepdim=True).float()
        want = (x.float() * count).to(x.dtype)
        ok = bool(torch.equal(back.x.view(torch.int16), want.view(torch.int16)))
        flags = [None] * world
        dist.all_gather_object(flags, ok, group=control_group)
        rows = torch.tensor([float(n_rows + c_valid)], dtype=torch.float64)
        dist.all_reduce(rows, op=dist.ReduceOp.SUM, group=control_group)
    bytes_per_step = float(rows.item()) * args.hidden * 2
    ordered = sorted(step_ms)
    return {
        "metric": "ep_dispatch_combine_payload_GBps", "value": bytes_per_step / (ms_per_step * 1e-3) / 1e9, "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (same generator and seeds as the ours arm)",
        "impl": "reference kernels, AOT stand-in, not the stock build",
        "what": "the reference's unmodified Python package, host runtime (peer.cu, pipeline.cu, epilogue wrappers, bindings) and kernel "
                "templates compiled for sm_100a; only its run-time JIT glue (csrc/jit.cpp) is replaced by static instantiations",
        "edits_to_reference_sources": "peer.cu:114-125 (owner lookup of mapped peer pointers and the three checks on it) removed: the lookup "
                                      "names the importing GPU on this driver and stops every multi-GPU run"
        if os.path.exists(os.path.join(str(refbuild.REF_OUT), "PEER_CHECKS_REMOVED")) else "none",
        "dispatch_us": disp_us, "combine_us": comb_us, "verified": all(flags),
        "step_ms_percentiles": {"p10": reduce_max(ordered[int(0.1 * len(ordered))]), "p50": reduce_max(ordered[len(ordered) // 2]),
                                "p90": reduce_max(ordered[min(len(ordered) - 1, int(0.9 * len(ordered)))])},
        "config": {"tokens_per_rank": args.tokens, "hidden": args.hidden, "experts": args.experts, "topk": args.topk,
                   "layout": "expanded", "alignment": args.alignment, "zero_padding": True, "parallelism": f"ep{world}"},
    }


def main():
    args = parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
    if "RANK" not in os.environ and args.gpus > 1:
        # convenience: re-launch under torch.distributed.run
        from nanoep_b200.testing.launcher import free_port

        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1",
               "--master-port", str(free_port()), os.path.abspath(__file__)] + sys.argv[1:]
        return subprocess.call(cmd)

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    os.environ.setdefault("LOCAL_RANK", str(local_rank))
    os.environ.setdefault("LOCAL_WORLD_SIZE", str(world))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world, timeout=timedelta(seconds=300), device_id=device)
    try:
        control = dist.new_group(backend="gloo", timeout=timedelta(seconds=300))
        runner = {"ours": run_ours, "nccl": run_nccl, "refkernels": run_refkernels}[args.impl]
        line = runner(args, rank, world, device, control)
        if rank == 0:
            print(json.dumps(line), flush=True)
        failed = line.get("verified") is False
    finally:
        dist.destroy_process_group()
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
