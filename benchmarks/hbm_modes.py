"""HBM bandwidth by access mix on one GPU: write-only, read-only, copy, and a 1:8 read:write row expansion.

The expert-major dispatch with zero padding writes ~12 bytes for every byte it reads, and the combine
reads ~8 bytes for every byte it writes, so a copy benchmark (1:1) is not the right ceiling for either.
This script measures the ceilings that are: library fill (write-only), library sum (read-only), library
copy, and `index_select` as a library row expansion of the dispatch's shape.  CUDA-event medians after
warm-up; every buffer is far larger than L2.

    python benchmarks/hbm_modes.py
"""

from __future__ import annotations

import json

import torch


def median_ms(fn, iters: int = 20, warmup: int = 5) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    for s, e in zip(starts, ends):
        s.record()
        fn()
        e.record()
    torch.cuda.synchronize()
    times = sorted(s.elapsed_time(e) for s, e in zip(starts, ends))
    return times[len(times) // 2]


def main() -> None:
    dev = torch.device("cuda", 0)
    nbytes = 1 << 30
    a = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    b = torch.empty_like(a)
    out = {}
    out["write_only_GBps"] = nbytes / median_ms(lambda: a.fill_(0)) / 1e6
    out["read_only_GBps"] = nbytes / median_ms(lambda: a.view(torch.float32).sum()) / 1e6
    out["copy_GBps_read_plus_write"] = 2 * nbytes / median_ms(lambda: b.copy_(a)) / 1e6
    # the headline dispatch's shape: 4096 rows of 7168 bf16 expanded into 48640 expert-major rows
    rows_in, rows_out, hidden = 4096, 48640, 7168
    x = torch.randn(rows_in, hidden, dtype=torch.bfloat16, device=dev)
    idx = torch.arange(rows_out, device=dev) % rows_in
    y = torch.empty(rows_out, hidden, dtype=torch.bfloat16, device=dev)
    ms = median_ms(lambda: torch.index_select(x, 0, idx, out=y))
    out["row_expansion_1_to_12_us"] = ms * 1e3
    out["row_expansion_GBps_read_plus_write"] = (rows_in + rows_out) * hidden * 2 / ms / 1e6
    print(json.dumps(out))


if __name__ == "__main__":
    main()
