"""Secondary benchmark configurations (run under torch.distributed.run, one process per GPU).

  --config skew     8192 tokens/rank x hidden 4096, 64 experts, top-6, Zipf(1.2) expert popularity under
                    a seeded permutation, 10% of the choices masked; compact layout; one fresh dispatch,
                    then the cached handle is reused for 10 dispatch/combine pairs with async_op=True.
  --config decode   tokens/rank in {1, 8, 32, 128, 512, 4096}, hidden 7168, 256 experts, top-8, uniform
                    routing; p50/p99 latency of fresh dispatch, cached dispatch and combine.
  --config published  the point of the reference's published figure: 256 tokens/rank, hidden 4096, top-8,
                    bf16, expert-major layout (the figure does not state the expert count; 256 is used).
                    Printed next to the reference's H20 numbers for the same GPU count.

Latencies are CUDA-event times on the caller's stream (max over ranks of each percentile); rank 0
prints one JSON line per measurement.  ``--impl nccl`` times torch.distributed all_to_all_single on
the same rows for comparison.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time
from datetime import timedelta
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--config", choices=("skew", "decode", "published"), required=True)
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--iters", type=int, default=50)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", choices=("ours", "nccl"), default="ours")
    p.add_argument("--tokens", type=str, default="1,8,32,128,512,4096")
    p.add_argument("--per-size-buffers", action="store_true",
                   help="decode: a buffer per token count (num_max_tokens_per_rank = tokens) instead of one sized for the largest")
    p.add_argument("--fused", type=str, default="",
                   help="decode/published: comma-separated dispatch_tokens:blocks[:fresh_tokens] settings of the single-launch dispatch paths to "
                        "measure one after the other (empty: the library defaults)")
    return p.parse_args()


def percentile(values, q):
    values = sorted(values)
    return values[min(len(values) - 1, int(round(q * (len(values) - 1))))]


def main():
    args = parse_args()
    import torch
    import torch.distributed as dist

    from nanoep_b200 import CudaBuffer, EPConfig
    from nanoep_b200.testing.cases import uniform_routing, zipf_routing

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29547")
    os.environ.setdefault("LOCAL_RANK", "0")
    os.environ.setdefault("LOCAL_WORLD_SIZE", str(world))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world, timeout=timedelta(seconds=300), device_id=device)
    control = dist.new_group(backend="gloo", timeout=timedelta(seconds=300))

    def reduce_max(v):
        t = torch.tensor([v], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=control)
        return float(t.item())

    def event_pair():
        return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def emit(record):
        if rank == 0:
            print(json.dumps(record), flush=True)

    try:
        if args.config == "skew":
            T, H, E, K = 8192, 4096, 64, 6
            idx, w = zipf_routing(T, E, K, seed=7 + rank, s=1.2, mask_fraction=0.1)
            x = torch.randn(T, H, generator=torch.Generator().manual_seed(rank)).to(torch.bfloat16).to(device)
            idx, w = idx.to(device), w.to(device)
            with CudaBuffer(control, EPConfig(E, K, H, T)) as buf:
                fresh_ms, pair_ms = [], []
                for it in range(args.warmup + args.iters):
                    torch.cuda.synchronize()
                    dist.barrier(group=control)
                    s0, e0 = event_pair()
                    s0.record()
                    got = buf.dispatch(x, topk_idx=idx, weights=w, async_op=True)
                    got.event.current_stream_wait()
                    e0.record()
                    s1, e1 = event_pair()
                    s1.record()
                    for _ in range(10):
                        again = buf.dispatch(x, handle=got.handle, weights=w, async_op=True)
                        again.event.current_stream_wait()
                        back = buf.combine(again.x, got.handle, async_op=True)
                        back.event.current_stream_wait()
                    e1.record()
                    torch.cuda.synchronize()
                    if it >= args.warmup:
                        fresh_ms.append(s0.elapsed_time(e0))
                        pair_ms.append(s1.elapsed_time(e1) / 10)
                buf.check_status()
                n = got.handle.layout.recv_count
                emit({"bench": "skew_cached", "n_gpus": world, "tokens_per_rank": T, "hidden": H, "experts": E, "topk": K,
                      "fresh_dispatch_us_p50": reduce_max(statistics.median(fresh_ms)) * 1e3,
                      "cached_dispatch_plus_combine_us_p50": reduce_max(statistics.median(pair_ms)) * 1e3,
                      "cached_dispatch_plus_combine_us_p99": reduce_max(percentile(pair_ms, 0.99)) * 1e3,
                      "recv_rows_rank0": n,
                      "payload_GBps_per_gpu": 2 * n * H * 2 / (statistics.median(pair_ms) * 1e-3) / 1e9})
        else:
            H, E, K = 7168, 256, 8
            sizes = [int(t) for t in args.tokens.split(",")]
            if args.config == "published":
                H, sizes = 4096, [256]
            from nanoep_b200.utils.build import load_extension

            ext = load_extension()
            settings = [tuple(int(v) for v in item.split(":")) for item in args.fused.split(",") if item] or [ext.fused_limits()]
            # one buffer for all sizes, or (--per-size-buffers) one per size with num_max_tokens_per_rank = that size, as a
            # server with a small maximum batch would configure it: the single-launch fresh dispatch sizes its outputs by
            # that maximum and is only used when the bound is modest
            groups = [[t] for t in sizes] if args.per_size_buffers else [sizes]
            for group_sizes in groups:
              with CudaBuffer(control, EPConfig(E, K, H, max(group_sizes))) as buf:
                for setting, T in ((s_, t_) for s_ in settings for t_ in group_sizes):
                    ext.set_fused_limits(*setting)
                    idx, w = uniform_routing(T, E, K, seed=3 + rank)
                    x = torch.randn(T, H, generator=torch.Generator().manual_seed(rank)).to(torch.bfloat16).to(device)
                    idx, w = idx.to(device), w.to(device)
                    if args.impl == "nccl":
                        flat = idx.flatten()
                        order = torch.argsort(flat, stable=True)
                        token_of = torch.arange(T, device=device).repeat_interleave(K)
                        send = x[token_of[order]]
                        counts = torch.bincount(flat, minlength=E).view(world, E // world).sum(1)
                        recv_counts = torch.empty_like(counts)
                        dist.all_to_all_single(recv_counts, counts)
                        ins, outs = counts.tolist(), recv_counts.tolist()
                        recv = torch.empty(sum(outs), H, dtype=x.dtype, device=device)
                        times = []
                        for it in range(args.warmup + args.iters):
                            s, e = event_pair()
                            s.record()
                            dist.all_to_all_single(recv, send, outs, ins)
                            e.record()
                            torch.cuda.synchronize()
                            if it >= args.warmup:
                                times.append(s.elapsed_time(e))
                        emit({"bench": "decode", "impl": "nccl_all_to_all_single (payload only, no routing)", "n_gpus": world, "tokens_per_rank": T,
                              "a2a_us_p50": reduce_max(statistics.median(times)) * 1e3, "a2a_us_p99": reduce_max(percentile(times, 0.99)) * 1e3})
                        continue
                    fresh, cached, comb, host_cached, host_comb = [], [], [], [], []
                    got = buf.dispatch(x, topk_idx=idx, weights=w, do_expand=True, alignment=1)
                    for it in range(args.warmup + args.iters):
                        dist.barrier(group=control)
                        a0, a1 = event_pair()
                        a0.record()
                        g = buf.dispatch(x, topk_idx=idx, weights=w, do_expand=True, alignment=1)
                        a1.record()
                        b0, b1 = event_pair()
                        b0.record()
                        h0 = time.perf_counter()
                        c = buf.dispatch(x, handle=got.handle, weights=w)
                        h1 = time.perf_counter()
                        b1.record()
                        c0, c1 = event_pair()
                        c0.record()
                        h2 = time.perf_counter()
                        back = buf.combine(c.x, got.handle)
                        h3 = time.perf_counter()
                        c1.record()
                        torch.cuda.synchronize()
                        if it >= args.warmup:
                            fresh.append(a0.elapsed_time(a1))
                            cached.append(b0.elapsed_time(b1))
                            comb.append(c0.elapsed_time(c1))
                            host_cached.append((h1 - h0) * 1e3)
                            host_comb.append((h3 - h2) * 1e3)
                    buf.check_status()
                    rec = {"bench": args.config, "impl": "ours", "n_gpus": world, "tokens_per_rank": T, "hidden": H,
                           "buffer_max_tokens": max(group_sizes),
                           "single_launch_limits": dict(zip(("dispatch_tokens", "blocks", "fresh_tokens"), ext.fused_limits()))}
                    if args.config == "published":
                        # reference figure (single-node H20): NanoEP / DeepEP 2.1.0 microseconds
                        published = {2: (69.4, 40.2, 51.9), 4: (78.5, 54.9, 70.4), 8: (147.1, 91.8, 102.5)}.get(world)
                        if published:
                            rec["reference_h20_us"] = dict(zip(("fresh_dispatch", "cached_dispatch", "combine"), published))
                    # host time spent inside the calls (enqueue only, no device wait): the floor of the event latencies
                    rec["host_call_us_p50"] = {"cached_dispatch": statistics.median(host_cached) * 1e3, "combine": statistics.median(host_comb) * 1e3}
                    for name, vals in (("fresh_dispatch", fresh), ("cached_dispatch", cached), ("combine", comb)):
                        rec[name + "_us_p50"] = reduce_max(statistics.median(vals)) * 1e3
                        rec[name + "_us_p99"] = reduce_max(percentile(vals, 0.99)) * 1e3
                    emit(rec)
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
