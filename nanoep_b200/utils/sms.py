"""How many SMs the communication kernels need to saturate NVLink.

The reference answers the same question with DeepEP's bandwidth model and Hopper per-SM constants
(nano_ep/backends/_sms.py:17-68).  The structure is kept (``num_sms=0`` means "use the estimate");
the per-SM constants are for B200 bulk-copy (TMA) rings, where one SM moves far more than a
load/store loop does, and the link rate comes from ``nvidia-smi nvlink -s`` or, when that is not
available, from the NVLink 5 figure of 900 GB/s per direction with the same 0.9 derate.
"""

from __future__ import annotations

import math
import re
import subprocess
from functools import cache

# One SM running a bulk-copy ring (5 warps x 3 stages of 14 KB rows): row bytes it moves per second when
# the rows cross NVLink.  Fitted to a sweep on 4 B200s (4096 x 7168 tokens per rank): 24 SMs sustain
# 425 GB/s of pulled rows and 350 GB/s of pushed rows; 48 SMs are within 6 % of all 148.
SM_BULK_READ_GBS = 17.0
SM_BULK_WRITE_GBS = 15.0
NVLINK_DERATE = 0.9
NVLINK5_PER_DIRECTION_GBS = 900.0


def _smi(*args: str) -> str:
    return subprocess.run(("nvidia-smi", *args), check=True, capture_output=True, text=True, timeout=5).stdout


def _norm_uuid(value: str) -> str:
    return value.strip().lower().removeprefix("gpu-").replace("-", "")


@cache
def nvlink_gbs(gpu_uuids: tuple[str, ...]) -> float:
    """Per-GPU one-direction NVLink rate (derated) if the whole group is NVLink-connected, else 0."""
    if len(gpu_uuids) < 2:
        return 0.0
    try:
        index_of = {}
        for line in _smi("--query-gpu=index,uuid", "--format=csv,noheader").splitlines():
            index, uuid = line.split(",", 1)
            index_of[_norm_uuid(uuid)] = f"GPU{index.strip()}"
        group = [index_of[_norm_uuid(u)] for u in gpu_uuids]
        topo = re.sub(r"\x1b\[[0-9;]*m", "", _smi("topo", "-m"))
        rows = [line.split() for line in topo.splitlines() if line.strip()]
        header = next(r for r in rows if len(r) >= 2 and all(re.fullmatch(r"GPU\d+", f) for f in r[:2]))
        columns = [f for f in header if re.fullmatch(r"GPU\d+", f)]
        links = {r[0]: dict(zip(columns, r[1:])) for r in rows if r is not header and r[0] in columns}
        for a in group:
            for b in group:
                if a != b and not links[a][b].startswith("NV"):
                    return 0.0
        per_gpu = dict.fromkeys(group, 0.0)
        current = None
        for line in _smi("nvlink", "-s").splitlines():
            if m := re.match(r"\s*GPU\s+(\d+):", line):
                current = f"GPU{m[1]}"
            elif current in per_gpu and (m := re.match(r"\s*Link\s+\d+:\s*([\d.]+)\s+GB/s", line)):
                per_gpu[current] += float(m[1])
        rate = min(per_gpu.values())
        # nvidia-smi reports the per-link rate as a bidirectional figure on some drivers; cap at NVLink 5.
        rate = min(rate, NVLINK5_PER_DIRECTION_GBS) if rate > 0 else NVLINK5_PER_DIRECTION_GBS
        return rate * NVLINK_DERATE
    except (OSError, subprocess.SubprocessError, KeyError, StopIteration, ValueError):
        return 0.0


def send_probability(world_size: int, num_experts: int, topk: int) -> float:
    """P(a token is sent to a given rank) for uniform routing over distinct experts."""
    local = num_experts // world_size
    return 1.0 - math.comb(num_experts - local, topk) / math.comb(num_experts, topk)


def theoretical_num_sms(device_sms: int, world_size: int, num_experts: int, topk: int, nvlink_bandwidth: float) -> int:
    """SM budget for the pull (dispatch) and push (combine) kernels; all SMs when NVLink is unknown."""
    if world_size == 1 or nvlink_bandwidth <= 0:
        return device_sms
    remote_fraction = 1.0 - 1.0 / world_size
    # Total row traffic an SM ring must sustain so that its NVLink share runs at link rate.
    traffic = nvlink_bandwidth / remote_fraction
    expected_ranks = world_size * send_probability(world_size, num_experts, topk)
    copies = max(1.0, topk / expected_ranks)  # expert-major layout: local stores per pulled row
    del copies  # local stores of the extra expert-major slots leave shared memory far faster than rows arrive
    need = traffic * max(
        1.0 / SM_BULK_READ_GBS,  # dispatch: bulk loads (remote + local)
        1.0 / SM_BULK_WRITE_GBS,  # combine: bulk stores to the sources
    )
    limit = device_sms // 2 * 2 or device_sms
    return max(4, min(4 * math.ceil(need * 1.3 / 4), limit))
