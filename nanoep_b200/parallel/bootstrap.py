"""Collective bootstrap helpers for the control plane.

The reference builds its buffer with a sequence of ``all_gather_object`` exchanges so that a local
failure on one rank is raised on *every* rank with the same aggregated message, followed by a
collective unmap -> free rollback (nano_ep/backends/cuda.py:103-229).  The same protocol is
expressed here as reusable steps so the CUDA buffer, the CPU buffer and the tests share it.
"""

from __future__ import annotations

import os
import socket
from dataclasses import asdict
from typing import Any, Callable

import torch.distributed as dist

from ..config import EPConfig


def gather_objects(group, obj: Any) -> list[Any]:
    world = dist.get_world_size(group=group)
    out: list[Any] = [None] * world
    dist.all_gather_object(out, obj, group=group)
    return out


def describe_error(exc: BaseException) -> str:
    return f"{type(exc).__name__}: {exc}"


def collective_step(group, what: str, fn: Callable[[], Any]) -> tuple[list[Any], list[str]]:
    """Run ``fn`` locally, exchange (value, error) and return all values plus ``rank r: error`` strings.

    Never raises for a local failure: the caller decides (after the exchange) so that all ranks take
    the same branch.
    """
    value, error = None, None
    try:
        value = fn()
    except Exception as exc:  # noqa: BLE001 - reported collectively
        error = describe_error(exc)
    results = gather_objects(group, {"value": value, "error": error})
    errors = [f"rank {r}: {res['error']}" for r, res in enumerate(results) if res["error"] is not None]
    return [res["value"] for res in results], errors


def local_facts(config: EPConfig, allow_multiple_reduction: bool, gpu_uuid: str | None) -> dict:
    if not isinstance(allow_multiple_reduction, bool):
        raise TypeError("allow_multiple_reduction must be bool")
    facts = {
        "config": asdict(config),
        "allow_multiple_reduction": allow_multiple_reduction,
        "hostname": socket.gethostname(),
        "gpu_uuid": gpu_uuid,
    }
    if "LOCAL_RANK" in os.environ:
        facts["local_rank"] = int(os.environ["LOCAL_RANK"])
    if "LOCAL_WORLD_SIZE" in os.environ:
        facts["local_world_size"] = int(os.environ["LOCAL_WORLD_SIZE"])
    return facts


def validate_group_facts(facts: list[dict], world_size: int, *, require_distinct_gpus: bool, hidden_multiple: int) -> None:
    """Cross-rank checks; identical inputs on every rank, so every rank raises the same error."""
    first = facts[0]
    if any(f["config"] != first["config"] for f in facts):
        raise ValueError("EPConfig mismatch across ranks")
    if any(f["allow_multiple_reduction"] != first["allow_multiple_reduction"] for f in facts):
        raise ValueError("allow_multiple_reduction mismatch across ranks")
    hosts = {f["hostname"] for f in facts}
    if len(hosts) != 1:
        raise ValueError(f"the buffer spans one node only, got hosts: {sorted(hosts)}")
    if require_distinct_gpus:
        uuids = [f["gpu_uuid"] for f in facts]
        if len(set(uuids)) != world_size:
            raise ValueError(f"Ranks must use distinct GPUs: {uuids}")
    if all("local_world_size" in f for f in facts):
        if any(f["local_world_size"] != world_size for f in facts):
            raise ValueError("Group must contain all local workers")
    if all("local_rank" in f for f in facts):
        local = sorted(f["local_rank"] for f in facts)
        if local != list(range(world_size)):
            raise ValueError(f"Invalid local rank assignment: {local}")
    cfg = first["config"]
    if world_size < 1 or world_size > 32 or world_size & (world_size - 1):
        raise ValueError("world size must be a power of two in [1, 32]")
    if cfg["num_experts"] % world_size != 0:
        raise ValueError("num_experts must be divisible by world_size")
    if cfg["hidden"] % hidden_multiple != 0:
        raise ValueError(f"hidden must be a positive multiple of {hidden_multiple}")
