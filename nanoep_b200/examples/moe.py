"""Forward MoE layer built on dispatch / combine, checked against a single-process evaluation.

    python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc-per-node=N \
        -m nanoep_b200.examples.moe [--layout compact] [--pattern skew] [--async-op] [--cached]

Every expert is a cheap element-wise map (a per-expert slope and offset through ``softsign``), so the
run time is communication.  Gate weights are applied by the experts: ``combine`` only sums.  The
command-line flags carry the names of the reference example (nano_ep/examples/moe.py:75-93) so that
scripts written for it keep working; ``--backend cpu`` runs the same flow on the Gloo/CPU backend.

The flow of one iteration:

1. a *producer* stream draws the tokens and the routing (seeded per rank and iteration) and records an
   event;
2. a *consumer* stream dispatches behind that event, evaluates the local experts on whatever layout
   came back, and combines;
3. the producer stream then allocates and poisons blocks of the sizes just used, so a result that the
   allocator handed back too early shows up as NaN in the final comparison.

When every iteration matches, rank 0 prints one ``NANOEP_MOE_OK=<json>`` line per rank.
"""

from __future__ import annotations

import argparse
import json
import os
from contextlib import nullcontext
from dataclasses import dataclass
from datetime import timedelta

import torch
import torch.distributed as dist

from nanoep_b200 import CpuBuffer, CudaBuffer, EPConfig

PATTERNS = ("mixed", "skew", "masked", "uneven")


# ----------------------------------------------------------------------------- experts
def expert_map(h: torch.Tensor, expert: torch.Tensor) -> torch.Tensor:
    """Row-wise expert: ``softsign(slope_e * h) + offset_e`` in FP32; ``expert`` holds one global id per row."""
    e = expert.to(torch.float32).unsqueeze(-1)
    slope = 0.5 + 0.25 * torch.remainder(e, 5.0)
    offset = 0.03125 * torch.remainder(e, 3.0)
    z = h.to(torch.float32) * slope
    return z / (1.0 + z.abs()) + offset


def rows_of_expert_major(handle, rows: int, device) -> tuple[torch.Tensor, torch.Tensor]:
    """Owner (local expert id) of every expert-major row and whether the row holds a token or padding."""
    offsets = handle.layout.expert_offsets.to(device)
    counts = handle.layout.expert_counts.to(device)
    sizes = offsets[1:] - offsets[:-1]
    owner = torch.repeat_interleave(torch.arange(sizes.numel(), device=device), sizes, output_size=rows)
    within = torch.arange(rows, device=device) - offsets[:-1][owner]
    return owner, within < counts[owner]


def run_local_experts(received) -> torch.Tensor:
    """Expert outputs in the layout ``combine`` expects: one row per slot (expert-major) or per receive row (compact)."""
    handle = received.handle
    per_rank = handle.config.num_experts // handle.world_size
    first = handle.rank * per_rank
    x = received.x
    if handle.do_expand:
        owner, live = rows_of_expert_major(handle, x.shape[0], x.device)
        out = expert_map(x, owner + first) * received.topk_weights.unsqueeze(-1)
        return torch.where(live.unsqueeze(-1), out, torch.zeros_like(out)).to(x.dtype)
    # compact: a receive row may feed several local experts; gather the (row, choice) pairs that are local
    row, choice = torch.nonzero(received.topk_idx >= 0, as_tuple=True)
    local = received.topk_idx[row, choice]
    part = expert_map(x[row], local + first) * received.topk_weights[row, choice].unsqueeze(-1)
    acc = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
    acc.index_add_(0, row, part)
    return acc.to(x.dtype)


def evaluate_without_ep(x, indices, weights, *, round_each_choice: bool) -> torch.Tensor:
    """The same layer on one device.  ``round_each_choice`` reproduces the expert-major data path, in which
    every choice travels back as its own bf16 row and the rows are summed in FP32 in ascending choice order."""
    acc = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
    for k in range(indices.shape[1]):
        chosen = indices[:, k]
        live = chosen >= 0
        term = expert_map(x, chosen.clamp(min=0)) * weights[:, k].unsqueeze(-1)
        if round_each_choice:
            term = term.to(x.dtype).to(torch.float32)
        acc += torch.where(live.unsqueeze(-1), term, torch.zeros_like(term))
    return acc.to(x.dtype)


# ----------------------------------------------------------------------------- inputs
def token_count(args, rank: int, world: int) -> int:
    if args.pattern != "uneven":
        return args.tokens
    # ragged ranks, and one rank that contributes nothing at all
    return 0 if rank == world - 1 else max(0, args.tokens - 5 * rank)


def draw_inputs(args, rank: int, world: int, iteration: int, device):
    """Tokens ~ N(0,1), distinct experts per token, positive gate weights; reproducible per (rank, iteration)."""
    gen = torch.Generator().manual_seed(7919 * (iteration + 1) + 104729 * rank + 13)
    T, K = token_count(args, rank, world), args.topk
    E = args.experts_per_rank * world
    x = torch.randn(T, args.hidden, generator=gen).to(torch.bfloat16)
    scores = torch.rand(T, E, generator=gen)
    if args.pattern == "skew":
        # everyone prefers the experts of rank 0: the first K columns win every top-k
        scores[:, : min(K, E)] += 2.0
    indices = scores.topk(K, dim=-1).indices.to(torch.int64)
    if args.pattern == "masked":
        indices = torch.full_like(indices, -1)
    else:
        indices = indices.masked_fill(torch.rand(T, K, generator=gen) < 0.15, -1)
    weights = torch.rand(T, K, generator=gen) * 0.9 + 0.1
    weights = weights / weights.sum(-1, keepdim=True)
    return x.to(device), indices.to(device), weights.to(device)


# ----------------------------------------------------------------------------- one rank
@dataclass
class Pending:
    """Results of one iteration, kept until the final comparison."""

    got: torch.Tensor
    want: torch.Tensor
    got_weights: torch.Tensor
    want_weights: torch.Tensor


class MoeRank:
    def __init__(self, args, rank: int, world: int, local_rank: int):
        self.args, self.rank, self.world = args, rank, world
        self.on_gpu = args.backend == "cuda"
        if self.on_gpu:
            torch.cuda.set_device(local_rank)
            self.device = torch.device("cuda", local_rank)
            self.producer, self.consumer = torch.cuda.Stream(), torch.cuda.Stream()
        else:
            self.device = torch.device("cpu")
            self.producer = self.consumer = None
        self.expanded = args.layout == "expanded"
        # the expert-major path without pre-reduction is reproducible bit for bit; the others round twice
        self.exact = self.expanded and not args.multiple_reduction
        self.handle = None
        self.pending: list[Pending] = []

    def on(self, stream):
        return torch.cuda.stream(stream) if self.on_gpu else nullcontext()

    def produce(self, iteration: int):
        with self.on(self.producer):
            x, indices, weights = draw_inputs(self.args, self.rank, self.world, iteration, self.device)
            want = evaluate_without_ep(x, indices, weights, round_each_choice=self.exact)
            want_weights = torch.where(indices >= 0, weights, torch.zeros_like(weights))
            ready = None
            if self.on_gpu:
                ready = torch.cuda.Event()
                ready.record()
        return x, indices, weights, want, want_weights, ready

    def consume(self, buffer, x, indices, weights, ready):
        args = self.args
        with self.on(self.consumer):
            fresh = self.handle is None
            received = buffer.dispatch(
                x,
                topk_idx=indices if fresh else None,
                weights=weights,
                handle=self.handle,
                do_expand=self.expanded if fresh else None,
                alignment=args.alignment if fresh else None,
                zero_padding=self.expanded,
                previous_event=ready,
                async_op=args.async_op,
            )
            if not fresh and received.handle is not self.handle:
                raise AssertionError("a cached dispatch must hand back the handle it was given")
            if received.event is not None:
                received.event.current_stream_wait()
            y = run_local_experts(received)
            combined = buffer.combine(y, received.handle, weights=received.topk_weights, async_op=args.async_op)
            if combined.event is not None:
                combined.event.current_stream_wait()
            if args.cached:
                self.handle = received.handle
        return combined, (y.shape, received.x.shape)

    def poison_recycled_blocks(self, shapes):
        """Ask the producer stream's allocator pool for blocks of the sizes the iteration just released."""
        if not self.on_gpu:
            return
        with torch.cuda.stream(self.producer):
            for shape in shapes:
                if shape[0] > 0:
                    torch.full(shape, float("nan"), dtype=torch.bfloat16, device=self.device)

    def verify(self):
        for it, p in enumerate(self.pending):
            if self.exact:
                if not torch.equal(p.got.view(torch.int16), p.want.view(torch.int16)):
                    worst = (p.got.float() - p.want.float()).abs().max().item()
                    raise AssertionError(f"iteration {it}: result differs from the single-process evaluation (max |diff| {worst})")
            else:
                torch.testing.assert_close(p.got.float(), p.want.float(), rtol=1e-2, atol=8e-3)
            if not torch.equal(p.got_weights, p.want_weights):
                raise AssertionError(f"iteration {it}: returned gate weights differ")

    def run(self, group):
        args = self.args
        config = EPConfig(self.world * args.experts_per_rank, args.topk, args.hidden, max(1, args.tokens))
        make_buffer = CudaBuffer if self.on_gpu else CpuBuffer
        with make_buffer(group, config, allow_multiple_reduction=args.multiple_reduction) as buffer:
            cached_inputs = None
            for iteration in range(args.iterations):
                x, indices, weights, want, want_weights, ready = self.produce(iteration)
                if args.cached:
                    # a cached handle replays the first iteration's routing: keep routing and weights, refresh the tokens
                    if cached_inputs is None:
                        cached_inputs = (indices, weights)
                    else:
                        indices, weights = cached_inputs
                        with self.on(self.producer):
                            want = evaluate_without_ep(x, indices, weights, round_each_choice=self.exact)
                            want_weights = torch.where(indices >= 0, weights, torch.zeros_like(weights))
                            if self.on_gpu:
                                ready = torch.cuda.Event()
                                ready.record()
                combined, shapes = self.consume(buffer, x, indices, weights, ready)
                self.pending.append(Pending(combined.x, want, combined.topk_weights, want_weights))
                del combined
                self.poison_recycled_blocks(shapes)
            if self.on_gpu:
                torch.cuda.synchronize()
                buffer.check_status()
            self.verify()
        return {"rank": self.rank, "world_size": self.world, "iterations": args.iterations, "exact": self.exact, **vars(args)}


# ----------------------------------------------------------------------------- command line
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
    p.add_argument("--pattern", choices=PATTERNS, default="mixed")
    p.add_argument("--async-op", action="store_true")
    p.add_argument("--cached", action="store_true")
    p.add_argument("--multiple-reduction", action="store_true")
    args = p.parse_args(argv)
    for name in ("hidden", "topk", "experts_per_rank", "alignment", "iterations"):
        if getattr(args, name) <= 0:
            p.error(f"--{name.replace('_', '-')} must be positive")
    if args.tokens < 0:
        p.error("--tokens must not be negative")
    if args.backend == "cuda" and args.hidden % CudaBuffer.HIDDEN_MULTIPLE:
        p.error(f"--hidden must be a multiple of {CudaBuffer.HIDDEN_MULTIPLE} on the CUDA backend")
    return args


@torch.no_grad()
def run(args):
    rank, world, local_rank = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    if int(os.environ.get("LOCAL_WORLD_SIZE", world)) != world:
        raise ValueError("all ranks of this example must run on one node")
    if args.topk > args.experts_per_rank * world:
        raise ValueError("--topk exceeds the number of experts")
    worker = MoeRank(args, rank, world, local_rank)
    dist.init_process_group("gloo", timeout=timedelta(seconds=90))
    try:
        report = worker.run(dist.group.WORLD)
        everyone = [None] * world if rank == 0 else None
        dist.gather_object(report, everyone, dst=0)
        for line in everyone or ():
            print("NANOEP_MOE_OK=" + json.dumps(line), flush=True)
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    run(parse_args())
