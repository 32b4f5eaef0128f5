"""Full expert-parallel SwiGLU MoE layer benchmark (and the grouped GEMM alone).

    python benchmarks/bench_moe.py --gpus 1 --gemm-only                       # tcgen05 grouped GEMM vs cuBLAS
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29541 \
        benchmarks/bench_moe.py --gpus 8                                      # fused layer vs unfused vs NCCL reference

Default shape is the DeepSeek-V3 one: 4096 tokens/rank, hidden 7168, intermediate 2048, 256 experts,
top-8, bf16, random-init weights ~N(0, 0.02), synthetic tokens.  Times are CUDA events on the
launching stream, median over steps, max over ranks.  The roofline of a fused path is the slower of
its FLOPs at the measured cuBLAS bf16 peak and its NVLink bytes at the measured peer bandwidth.
One JSON line per arm is printed by rank 0.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
from datetime import timedelta
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

PEER_GBS = 770.0  # measured peer copy bandwidth per direction on this pool


def measured_peaks():
    path = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return float(data["bf16_tflops"]), float(data["bf16_tflops_sustained"]), float(data["hbm_gbs"]), "measured"
    return 1590.0, 1400.0, 6650.0, "fallback"


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--tokens", type=int, default=4096)
    p.add_argument("--hidden", type=int, default=7168)
    p.add_argument("--inter", type=int, default=2048)
    p.add_argument("--experts", type=int, default=256)
    p.add_argument("--topk", type=int, default=8)
    p.add_argument("--gemm-only", action="store_true")
    p.add_argument("--arms", default="fused,fused_combine,unfused,nccl")
    return p.parse_args()


def timed(fn, steps, warmup, flush):
    import torch

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for i in range(steps):
        flush.fill_(i & 0xFF)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    return times


def gemm_only(args, device):
    import torch

    from nanoep_b200.ops import grouped_gemm as gg

    burst, sustained, _, basis = measured_peaks()
    local = max(1, args.experts // 8)  # experts one rank of an EP8 group owns
    rows_per = max(128, (args.tokens * args.topk // local + 127) // 128 * 128)
    offsets = torch.arange(local + 1, dtype=torch.int64, device=device) * rows_per
    rows = rows_per * local
    torch.manual_seed(0)
    a = (torch.randn(rows, args.hidden, device=device) * 0.5).to(torch.bfloat16)
    w13 = (torch.randn(local, 2 * args.inter, args.hidden, device=device) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(local, args.hidden, args.inter, device=device) * 0.02).to(torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    h = gg.grouped_gemm(a, w13, offsets, swiglu=True)
    out = {}
    for name, fn, flops in (
        ("up_swiglu", lambda: gg.grouped_gemm(a, w13, offsets, swiglu=True), 2.0 * rows * args.hidden * 2 * args.inter),
        ("up_swiglu_3stage", lambda: gg.grouped_gemm(a, w13, offsets, swiglu=True, stages=3), 2.0 * rows * args.hidden * 2 * args.inter),
        ("up_swiglu_pair", lambda: gg.grouped_gemm(a, w13, offsets, swiglu=True, pair=True), 2.0 * rows * args.hidden * 2 * args.inter),
        ("down_pair", lambda: gg.grouped_gemm(h, w2, offsets, pair=True), 2.0 * rows * args.hidden * args.inter),
        ("down", lambda: gg.grouped_gemm(h, w2, offsets), 2.0 * rows * args.hidden * args.inter),
        ("down_3stage", lambda: gg.grouped_gemm(h, w2, offsets, stages=3), 2.0 * rows * args.hidden * args.inter),
        ("cublas_up", lambda: torch.bmm(a.view(local, rows_per, args.hidden), w13.transpose(1, 2)), 2.0 * rows * args.hidden * 2 * args.inter),
        ("cublas_down", lambda: torch.bmm(h.view(local, rows_per, args.inter), w2.transpose(1, 2)), 2.0 * rows * args.hidden * args.inter),
    ):
        ms = statistics.median(timed(fn, args.steps, args.warmup, flush))
        out[name] = {"ms": ms, "tflops": flops / ms / 1e9, "frac_of_burst_peak": flops / ms / 1e9 / burst}
    gg.check_status()
    print(json.dumps({"bench": "grouped_gemm", "rows": rows, "experts": local, "hidden": args.hidden, "inter": args.inter,
                      "peak_basis": basis, "bf16_tflops_burst": burst, **out}))


def run(args):
    import torch
    import torch.distributed as dist

    from nanoep_b200 import CudaBuffer, EPConfig
    from nanoep_b200.models.moe_layer import ExpertParallelMoE
    from nanoep_b200.ops import grouped_gemm as gg
    from nanoep_b200.testing.cases import balanced_routing

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29543")
    os.environ.setdefault("LOCAL_RANK", "0")
    os.environ.setdefault("LOCAL_WORLD_SIZE", str(world))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if args.gemm_only:
        return gemm_only(args, device)
    dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world, timeout=timedelta(seconds=300), device_id=device)
    try:
        control = dist.new_group(backend="gloo", timeout=timedelta(seconds=300))
        burst, sustained, _, basis = measured_peaks()
        T, H, I, E, K = args.tokens, args.hidden, args.inter, args.experts, args.topk
        L = E // world
        torch.manual_seed(1000 + rank)
        x = (torch.randn(T, H, device=device)).to(torch.bfloat16)
        idx, w = balanced_routing(T, E, K, seed=99 + rank)
        idx, w = idx.to(device), w.to(device)
        w13 = (torch.randn(L, 2 * I, H, device=device) * 0.02).to(torch.bfloat16)
        w2 = (torch.randn(L, H, I, device=device) * 0.02).to(torch.bfloat16)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)

        def reduce_max(v):
            t = torch.tensor([v], dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=control)
            return float(t.item())

        def reduce_sum(v):
            t = torch.tensor([v], dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=control)
            return float(t.item())

        results = []
        with CudaBuffer(control, EPConfig(E, K, H, T)) as buf:
            layers = {
                "fused": ExpertParallelMoE(buf, w13, w2, fuse_combine=True, overlap_dispatch=True),
                "fused_combine": ExpertParallelMoE(buf, w13, w2, fuse_combine=True, overlap_dispatch=False),
                "fused_serialized": ExpertParallelMoE(buf, w13, w2, fuse_combine=True, overlap_dispatch=True),
                "unfused": ExpertParallelMoE(buf, w13, w2, fuse_combine=False, overlap_dispatch=False),
            }
            layers["fused_serialized"].serialize_overlap = True
            probe = layers["unfused"]
            probe(x, idx, w)
            torch.cuda.synchronize()
            handle = probe.last_handle
            rows_valid = int(handle.layout.expert_counts.sum().item())
            rows_padded = handle.layout.expanded_capacity
            n_recv = handle.layout.recv_count
            remote_rows = n_recv - int((handle.layout.recv_metadata[:, 0] == rank).sum().item())
            flops = 2.0 * rows_padded * H * 3 * I  # what the tensor cores execute (padding included)
            useful = 2.0 * rows_valid * H * 3 * I
            nvlink_bytes = (remote_rows + rows_valid * (world - 1) / world) * H * 2  # dispatch in + combine out
            for name in args.arms.split(","):
                if name == "nccl":
                    continue
                layer = layers[name]
                dist.barrier(group=control)
                ms = reduce_max(statistics.median(timed(lambda: layer(x, idx, w), args.steps, args.warmup, flush)))
                buf.check_status()
                gg.check_status()
                layer.profile = True
                layer(x, idx, w)
                layer(x, idx, w)
                layer.profile = False
                profile = {k: reduce_max(v) for k, v in layer.last_profile.items()}
                t_compute = reduce_max(flops / (burst * 1e12)) * 1e3
                t_link = reduce_max(nvlink_bytes / (PEER_GBS * 1e9)) * 1e3 if world > 1 else 0.0
                results.append({
                    "bench": "moe_layer", "impl": name, "n_gpus": world, "ms_per_layer": ms,
                    "tokens_per_s": reduce_sum(T) / (ms * 1e-3),
                    "tflops_executed_per_gpu": flops / ms / 1e9, "tflops_useful_per_gpu": useful / ms / 1e9,
                    "roofline_ms": max(t_compute, t_link), "roofline_frac": max(t_compute, t_link) / ms,
                    "roofline_terms_ms": {"compute_at_burst_peak": t_compute, "nvlink_at_770GBs": t_link}, "peak_basis": basis,
                    "rows": {"valid": rows_valid, "padded": rows_padded, "recv_dedup": n_recv},
                    "steps_us": profile,
                })
        if "nccl" in args.arms.split(","):
            nccl = dist.group.WORLD

            def nccl_layer():
                flat = idx.flatten()
                token_of = torch.arange(T, device=device).repeat_interleave(K)
                order = torch.argsort(flat, stable=True)
                send = x[token_of[order]]
                per_expert = torch.bincount(flat, minlength=E)
                send_counts = per_expert.view(world, L).sum(1)
                recv_counts = torch.empty_like(send_counts)
                dist.all_to_all_single(recv_counts, send_counts, group=nccl)
                recv_expert = torch.empty(world * L, dtype=per_expert.dtype, device=device)
                dist.all_to_all_single(recv_expert, per_expert, group=nccl)
                ins, outs = send_counts.tolist(), recv_counts.tolist()
                recv = torch.empty(sum(outs), H, dtype=x.dtype, device=device)
                dist.all_to_all_single(recv, send, outs, ins, group=nccl)
                expert_of = torch.repeat_interleave(torch.arange(L, device=device).repeat(world), recv_expert)
                perm = torch.argsort(expert_of, stable=True)
                xin = recv[perm]
                counts = torch.bincount(expert_of, minlength=L).tolist()
                y = torch.empty_like(xin)
                at = 0
                for e, c in enumerate(counts):
                    if c:
                        gu = xin[at:at + c] @ w13[e].t()
                        hmid = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
                        y[at:at + c] = hmid @ w2[e].t()
                    at += c
                back = torch.empty_like(recv)
                back[perm] = y
                ret = torch.empty(T * K, H, dtype=x.dtype, device=device)
                dist.all_to_all_single(ret, back, ins, outs, group=nccl)
                out = torch.zeros(T, H, dtype=torch.float32, device=device)
                out.index_add_(0, token_of[order], ret.float() * w.flatten()[order, None])
                return out.to(x.dtype)

            dist.barrier(group=control)
            ms = reduce_max(statistics.median(timed(nccl_layer, args.steps, args.warmup, flush)))
            results.append({"bench": "moe_layer", "impl": "nccl_all_to_all+per_expert_matmul", "n_gpus": world, "ms_per_layer": ms,
                            "tokens_per_s": reduce_sum(T) / (ms * 1e-3)})
        if rank == 0:
            for r in results:
                print(json.dumps(r), flush=True)
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    run(parse_args())
