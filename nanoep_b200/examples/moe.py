"""Forward-only MoE over dispatch/combine:

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node=N -m nanoep_b200.examples.moe [--async-op --cached]

Experts are distinct element-wise transforms so the example stays a communication example; gate
weights are applied before combine (combine only sums).  Inputs are produced on a separate producer
stream and handed over with ``previous_event``; with ``--async-op`` the consumer waits on the result
event only.  The same flags as the reference example (nano_ep/examples/moe.py:75-93) plus
``--backend cpu`` to run the identical flow on the Gloo/CPU backend without a GPU.
Each rank prints ``NANOEP_MOE_OK=<json>`` through rank 0 when its results match a dense reference.
"""

from __future__ import annotations

import argparse
import contextlib
import json
import os
from datetime import timedelta

import torch
import torch.distributed as dist

from nanoep_b200 import CpuBuffer, CudaBuffer, EPConfig


def _expert_fn(x_fp32, global_expert):
    g = global_expert[:, None].float()
    return torch.tanh(x_fp32 * (1 + g / 32) + g / 64)


def expert_forward(received):
    """Evaluate the local experts from the receive metadata (handles padding in the expert-major layout)."""
    handle = received.handle
    local_experts = handle.config.num_experts // handle.world_size
    base = handle.rank * local_experts
    x = received.x.float()
    if handle.do_expand:
        layout = handle.layout
        rows = torch.arange(x.shape[0], device=x.device)
        expert = torch.bucketize(rows, layout.expert_offsets[1:].to(x.device), right=True).clamp(max=local_experts - 1)
        valid = rows < (layout.expert_offsets[:-1] + layout.expert_counts).to(x.device)[expert]
        value = _expert_fn(x, expert + base) * received.topk_weights[:, None]
        return value.masked_fill(~valid[:, None], 0).to(received.x.dtype)
    value = torch.zeros_like(x)
    for k in range(handle.config.num_topk):
        expert = received.topk_idx[:, k]
        contribution = _expert_fn(x, expert + base) * received.topk_weights[:, k, None]
        value += contribution.masked_fill((expert < 0)[:, None], 0)
    return value.to(received.x.dtype)


def dense_reference(x, indices, weights):
    result = torch.zeros_like(x, dtype=torch.float32)
    for k in range(indices.shape[1]):
        expert = indices[:, k]
        value = _expert_fn(x.float(), expert)
        result += (value * weights[:, k, None]).masked_fill((expert < 0)[:, None], 0)
    return result.to(x.dtype)


def make_inputs(args, rank, size, iteration, device):
    tokens = args.tokens
    if args.pattern == "uneven":
        tokens = 0 if rank == size - 1 else max(0, tokens - rank * 3)
    row = torch.arange(tokens, device=device)
    col = torch.arange(args.hidden, device=device)
    x = (((row[:, None] * 7 + col + rank * 11 + iteration * 3) % 127 - 63) / 64).to(torch.bfloat16)
    experts = args.experts_per_rank * size
    base = torch.zeros_like(row) if args.pattern == "skew" else row + rank * args.experts_per_rank
    indices = ((base[:, None] + torch.arange(args.topk, device=device)) % experts).clone()
    if args.pattern == "masked":
        indices.fill_(-1)
    else:
        indices[:, -1].masked_fill_(row % 7 == 0, -1)
    weights = ((row[:, None] + torch.arange(args.topk, device=device) + iteration) % 5 + 1).float() / (5 * args.topk)
    return x.contiguous(), indices.contiguous(), weights.contiguous()


def parse_args(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--backend", choices=("cuda", "cpu"), default="cuda")
    p.add_argument("--layout", choices=("compact", "expanded"), default="expanded")
    p.add_argument("--dtype", choices=("bf16",), default="bf16")
    p.add_argument("--tokens", type=int, default=129)
    p.add_argument("--hidden", type=int, default=1024)
    p.add_argument("--topk", type=int, default=3)
    p.add_argument("--experts-per-rank", type=int, default=8)
    p.add_argument("--alignment", type=int, default=16)
    p.add_argument("--iterations", type=int, default=4)
    p.add_argument("--pattern", choices=("mixed", "skew", "masked", "uneven"), default="mixed")
    p.add_argument("--async-op", action="store_true")
    p.add_argument("--cached", action="store_true")
    p.add_argument("--multiple-reduction", action="store_true")
    args = p.parse_args(argv)
    if args.tokens < 0 or min(args.hidden, args.topk, args.experts_per_rank, args.alignment, args.iterations) <= 0:
        p.error("tokens must be nonnegative; other dimensions/iterations must be positive")
    if args.backend == "cuda" and args.hidden % 256 != 0:
        p.error("hidden must be a multiple of 256")
    return args


@torch.no_grad()
def run(args):
    rank, size, local = (int(os.environ[name]) for name in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    if int(os.environ.get("LOCAL_WORLD_SIZE", size)) != size:
        raise ValueError("This example requires a single node")
    cuda = args.backend == "cuda"
    if cuda:
        torch.cuda.set_device(local)
    device = "cuda" if cuda else "cpu"
    dist.init_process_group("gloo", timeout=timedelta(seconds=90))
    try:
        cfg = EPConfig(size * args.experts_per_rank, args.topk, args.hidden, max(1, args.tokens))
        stream_ctx = torch.cuda.stream if cuda else (lambda s: contextlib.nullcontext())
        producer, consumer = (torch.cuda.Stream(), torch.cuda.Stream()) if cuda else (None, None)
        buffer_cls = CudaBuffer if cuda else CpuBuffer
        checks, handle = [], None
        with buffer_cls(dist.group.WORLD, cfg, allow_multiple_reduction=args.multiple_reduction) as buffer:
            for iteration in range(args.iterations):
                with stream_ctx(producer):
                    x, indices, weights = make_inputs(args, rank, size, iteration, device)
                    expected = dense_reference(x, indices, weights)
                    expected_weights = weights.masked_fill(indices < 0, 0)
                    ready = None
                    if cuda:
                        ready = torch.cuda.Event()
                        ready.record()
                with stream_ctx(consumer):
                    received = buffer.dispatch(
                        x, topk_idx=indices if handle is None else None, weights=weights, handle=handle,
                        do_expand=args.layout == "expanded", alignment=args.alignment,
                        zero_padding=args.layout == "expanded", previous_event=ready, async_op=args.async_op,
                    )
                    if handle is not None and received.handle is not handle:
                        raise AssertionError("cached dispatch must preserve handle identity")
                    if received.event is not None:
                        received.event.current_stream_wait()
                    y = expert_forward(received)
                    result = buffer.combine(y, received.handle, weights=received.topk_weights, async_op=args.async_op)
                    if result.event is not None:
                        result.event.current_stream_wait()
                    checks.append((result.x, expected, result.topk_weights, expected_weights))
                    if args.cached:
                        handle = received.handle
                del x, indices, weights, y, received, result
                if cuda:
                    # reuse producer allocations while communication/consumer work may still be pending
                    with torch.cuda.stream(producer):
                        churn = torch.empty((max(1, args.tokens), args.hidden), device="cuda", dtype=expected.dtype)
                        churn.fill_(-77)
                        del churn
            if cuda:
                torch.cuda.synchronize()
                buffer.check_status()
            for actual, expected, actual_weights, expected_weights in checks:
                torch.testing.assert_close(actual, expected, rtol=0.03, atol=0.03)
                torch.testing.assert_close(actual_weights, expected_weights, rtol=0, atol=0)
        reports = [None] * size if rank == 0 else None
        dist.gather_object({"rank": rank, "world_size": size, **vars(args)}, reports, dst=0)
        if rank == 0:
            for report in reports:
                print("NANOEP_MOE_OK=" + json.dumps(report), flush=True)
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    run(parse_args())
