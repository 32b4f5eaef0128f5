"""One rank of the fused MoE layer test (torch.distributed.run, one GPU per rank; also runs with 1 rank)."""

import os
import sys
from datetime import timedelta

import torch
import torch.distributed as dist

from nanoep_b200 import CudaBuffer, EPConfig
from nanoep_b200.models.moe_layer import ExpertParallelMoE, dense_reference
from nanoep_b200.ops import grouped_gemm as gg
from nanoep_b200.testing.cases import balanced_routing, zipf_routing


def main():
    rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    torch.cuda.set_device(local)
    dist.init_process_group("gloo", timeout=timedelta(seconds=120))
    try:
        T, H, I, E, K = 333, 512, 256, 8 * world, 4
        L = E // world
        gen = torch.Generator().manual_seed(7)
        w13_all = (torch.randn(E, 2 * I, H, generator=gen) * 0.06).to(torch.bfloat16).cuda()
        w2_all = (torch.randn(E, H, I, generator=gen) * 0.06).to(torch.bfloat16).cuda()
        cfg = EPConfig(E, K, H, T)
        with CudaBuffer(dist.group.WORLD, cfg) as buf:
            for variant, (fuse, overlap) in enumerate([(False, False), (True, False), (False, True), (True, True)]):
                layer = ExpertParallelMoE(buf, w13_all[rank * L:(rank + 1) * L].contiguous(), w2_all[rank * L:(rank + 1) * L].contiguous(),
                                          fuse_combine=fuse, overlap_dispatch=overlap)
                for it, routing in enumerate((balanced_routing, zipf_routing)):
                    idx, w = routing(T - rank, E, K, seed=31 * it + rank)
                    x = (torch.randn(T - rank, H, generator=torch.Generator().manual_seed(100 + rank + it)) * 0.5).to(torch.bfloat16)
                    x, idx, w = x.cuda(), idx.cuda(), w.cuda()
                    out = layer(x, idx, w)
                    torch.cuda.synchronize()
                    buf.check_status()
                    gg.check_status()
                    ref = dense_reference(x, idx, w, w13_all, w2_all)
                    torch.testing.assert_close(out.float(), ref.float(), rtol=1e-2, atol=4e-3)
                    # cached routing through the layer
                    out2 = layer(x, None, w, handle=layer.last_handle)
                    torch.cuda.synchronize()
                    torch.testing.assert_close(out2.float(), ref.float(), rtol=1e-2, atol=4e-3)
        dist.barrier()
        print(f"NANOEP_MOE_LAYER_OK={rank}", flush=True)
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())
