"""Fused SwiGLU MoE layer on N GPUs, checked against a dense PyTorch reference:

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node=N -m nanoep_b200.examples.fused_moe [--tokens 512 --hidden 1024 --inter 512]

dispatch (expert-major, 128-row alignment, zero padding) -> tcgen05 grouped GEMM with SwiGLU epilogue
-> down-projection GEMM whose epilogue applies the gate weight and bulk-stores rows into the source
ranks' return partitions -> peer barrier + FP32 reduction.  Prints ``NANOEP_FUSED_MOE_OK=<rank>``.
"""

from __future__ import annotations

import argparse
import os
from datetime import timedelta

import torch
import torch.distributed as dist

from nanoep_b200 import CudaBuffer, EPConfig
from nanoep_b200.models.moe_layer import ExpertParallelMoE, dense_reference
from nanoep_b200.ops import grouped_gemm as gg
from nanoep_b200.testing.cases import balanced_routing


def main():
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--tokens", type=int, default=512)
    p.add_argument("--hidden", type=int, default=1024)
    p.add_argument("--inter", type=int, default=512)
    p.add_argument("--experts-per-rank", type=int, default=8)
    p.add_argument("--topk", type=int, default=4)
    args = p.parse_args()
    rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    torch.cuda.set_device(local)
    dist.init_process_group("gloo", timeout=timedelta(seconds=120))
    try:
        E, L = args.experts_per_rank * world, args.experts_per_rank
        gen = torch.Generator().manual_seed(0)  # every rank builds all experts' weights to check against
        w13 = (torch.randn(E, 2 * args.inter, args.hidden, generator=gen) * 0.05).to(torch.bfloat16).cuda()
        w2 = (torch.randn(E, args.hidden, args.inter, generator=gen) * 0.05).to(torch.bfloat16).cuda()
        x = (torch.randn(args.tokens, args.hidden, generator=torch.Generator().manual_seed(1 + rank)) * 0.5).to(torch.bfloat16).cuda()
        idx, w = balanced_routing(args.tokens, E, args.topk, seed=10 + rank, device="cuda")
        with CudaBuffer(dist.group.WORLD, EPConfig(E, args.topk, args.hidden, args.tokens)) as buf:
            layer = ExpertParallelMoE(buf, w13[rank * L:(rank + 1) * L].contiguous(), w2[rank * L:(rank + 1) * L].contiguous())
            out = layer(x, idx, w)
            torch.cuda.synchronize()
            buf.check_status()
            gg.check_status()
        torch.testing.assert_close(out.float(), dense_reference(x, idx, w, w13, w2).float(), rtol=3e-2, atol=3e-2)
        dist.barrier()
        print(f"NANOEP_FUSED_MOE_OK={rank}", flush=True)
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
