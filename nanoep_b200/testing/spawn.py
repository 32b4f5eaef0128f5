"""Run a function on N Gloo ranks (CPU child processes) and re-raise the first failure."""

from __future__ import annotations

import multiprocessing as mp
import os
import traceback
from datetime import timedelta

from .launcher import free_port


def _entry(rank, world, port, target, args, queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), LOCAL_WORLD_SIZE=str(world), OMP_NUM_THREADS="1")
    import torch
    import torch.distributed as dist

    torch.set_num_threads(1)
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=60))
        try:
            result = target(rank, world, *args)
        finally:
            dist.destroy_process_group()
        queue.put((rank, None, result))
    except BaseException:  # noqa: BLE001 - shipped to the parent
        queue.put((rank, traceback.format_exc(), None))


def run_gloo(world: int, target, *args, timeout: float = 120):
    """``target(rank, world, *args)`` must be importable (module-level). Returns results by rank."""
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, target, args, queue), daemon=True) for r in range(world)]
    for p in procs:
        p.start()
    results, errors = {}, []
    try:
        for _ in range(world):
            rank, err, value = queue.get(timeout=timeout)
            if err:
                errors.append(f"rank {rank}:\n{err}")
            results[rank] = value
    finally:
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
    if errors:
        raise AssertionError("\n".join(errors))
    return [results[r] for r in range(world)]
