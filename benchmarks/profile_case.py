"""Small, self-terminating workloads for kernel profilers (one GPU, a few GB at most).

    python benchmarks/profile_case.py ep      # 2 logical ranks on one GPU: stage, plan, pull, combine (+ single-rank local_combine)
    python benchmarks/profile_case.py gemm    # tcgen05 grouped GEMM: SwiGLU up-projection, down-projection, scatter variant inputs

Inputs are larger than L2 (126 MB) so DRAM figures are meaningful; each kernel of interest runs a
handful of times.  Meant to be run once plainly and then once per kernel under
``ncu --set full --clock-control none -k regex:<one kernel name> -s 1 -c 1`` (one kernel per capture).
"""

import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from nanoep_b200 import EmulatedGroup, EPConfig  # noqa: E402
from nanoep_b200.ops import grouped_gemm as gg  # noqa: E402
from nanoep_b200.testing.cases import balanced_routing  # noqa: E402


def run_ep():
    T, H, E, K = 2048, 7168, 64, 8
    for world in (2, 1):
        cfg = EPConfig(E, K, H, T)
        xs = [torch.randn(T, H, device="cuda").to(torch.bfloat16) for _ in range(world)]
        routing = [balanced_routing(T, E, K, seed=5 + r, device="cuda") for r in range(world)]
        idx, w = [r[0] for r in routing], [r[1] for r in routing]
        with EmulatedGroup(world, cfg) as group:
            for _ in range(2):
                got = group.dispatch(xs, topk_idx=idx, weights=w, do_expand=True, alignment=128, zero_padding=True, num_sms=148 // world)
                back = group.combine([g.x for g in got], [g.handle for g in got], num_sms=148 // world)
            torch.cuda.synchronize()
            group.check_status()
            print("ep world", world, "rows", [g.handle.layout.recv_count for g in got], "capacity", [g.handle.layout.expanded_capacity for g in got])


def run_gemm():
    experts, rows_per, H, I = 8, 1024, 7168, 2048
    offsets = torch.arange(experts + 1, dtype=torch.int64, device="cuda") * rows_per
    a = (torch.randn(experts * rows_per, H, device="cuda") * 0.5).to(torch.bfloat16)
    w13 = (torch.randn(experts, 2 * I, H, device="cuda") * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(experts, H, I, device="cuda") * 0.02).to(torch.bfloat16)
    for _ in range(2):
        h = gg.grouped_gemm(a, w13, offsets, swiglu=True)
        y = gg.grouped_gemm(h, w2, offsets)
    for _ in range(2):  # CTA-pair kernels (tcgen05 cta_group::2)
        h = gg.grouped_gemm(a, w13, offsets, swiglu=True, pair=True)
        y = gg.grouped_gemm(h, w2, offsets, pair=True)
    torch.cuda.synchronize()
    gg.check_status()
    print("gemm rows", a.shape[0], "flops up", 2 * a.shape[0] * H * 2 * I, "down", 2 * a.shape[0] * H * I)


if __name__ == "__main__":
    {"ep": run_ep, "gemm": run_gemm}[sys.argv[1]]()
