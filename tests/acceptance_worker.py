"""One rank of the acceptance run: every delivery profile of the forward MoE example in ONE process group.

The profiles cover what the reference's acceptance tier covers (tests/distributed/test_acceptance.py:17-28):
both receive layouts, the four routing patterns, small and DeepSeek-size rows (256 tokens x 7168 x top-8),
synchronous and asynchronous + cached operation.  Running them in one launch keeps the GPU time to the
operations themselves instead of ten interpreter start-ups per rank.
"""

import os
import sys
from datetime import timedelta

import torch
import torch.distributed as dist

from nanoep_b200.examples.moe import MoeRank, parse_args

PROFILES = {
    "small-compact": ["--layout", "compact", "--tokens", "17", "--hidden", "256", "--iterations", "3"],
    "small-expanded": ["--layout", "expanded", "--tokens", "17", "--hidden", "256", "--iterations", "3"],
    "wide-compact": ["--layout", "compact", "--tokens", "256", "--hidden", "4096", "--topk", "8", "--iterations", "4", "--async-op", "--cached"],
    "wide-expanded": ["--layout", "expanded", "--tokens", "256", "--hidden", "7168", "--topk", "8", "--iterations", "8", "--async-op", "--cached"],
    "hot-experts-compact": ["--layout", "compact", "--pattern", "skew", "--iterations", "16", "--async-op", "--cached"],
    "hot-experts-expanded": ["--layout", "expanded", "--pattern", "skew", "--iterations", "16", "--async-op", "--cached"],
    "all-masked-compact": ["--layout", "compact", "--pattern", "masked", "--tokens", "33", "--hidden", "256", "--async-op", "--cached"],
    "all-masked-expanded": ["--layout", "expanded", "--pattern", "masked", "--tokens", "33", "--hidden", "256", "--async-op", "--cached"],
    "ragged-compact": ["--layout", "compact", "--pattern", "uneven", "--tokens", "65", "--iterations", "8", "--async-op", "--cached"],
    "ragged-expanded": ["--layout", "expanded", "--pattern", "uneven", "--tokens", "65", "--iterations", "8", "--async-op", "--cached"],
    "pre-reduced-expanded": ["--layout", "expanded", "--multiple-reduction", "--tokens", "129", "--topk", "4", "--iterations", "4"],
}


@torch.no_grad()
def main():
    rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    backend = os.environ.get("NANOEP_ACCEPT_BACKEND", "cuda")
    only = [n for n in os.environ.get("NANOEP_ACCEPT_PROFILES", "").split(",") if n]
    dist.init_process_group("gloo", timeout=timedelta(seconds=180))
    try:
        for name, flags in PROFILES.items():
            if only and name not in only:
                continue
            args = parse_args(["--backend", backend, *flags])
            MoeRank(args, rank, world, local).run(dist.group.WORLD)
            dist.barrier()
            print(f"NANOEP_ACCEPT_OK={name} rank={rank}", flush=True)
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())
