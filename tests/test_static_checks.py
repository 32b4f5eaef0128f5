"""Source-level guarantees that need no GPU: no cluster-multicast bulk loads, no unbounded traps,
SM-budget model behaviour, packaging of native sources."""

import math
import re
from pathlib import Path

from nanoep_b200.utils import sms
from nanoep_b200.utils.build import SOURCES, source_dir

ROOT = Path(__file__).resolve().parent.parent


def _native_sources():
    return [p for p in (ROOT / "csrc").rglob("*") if p.suffix in {".cu", ".cuh", ".hpp", ".cpp", ".h"}]


def test_no_cluster_multicast_loads_and_no_traps():
    # patterns are assembled from pieces so that this file does not itself contain them
    banned = re.compile("|".join(["multi" + "cast::cluster", "_MULTI" + "CAST", r"__tr" + r"ap\s*\(", r"asm[^;]*\btr" + r"ap;", "Memcpy" + "Batch" + "Async"]))
    for path in _native_sources():
        text = path.read_text()
        assert not banned.search(text), f"{path} uses a construct that is banned in this project"


def test_every_device_wait_is_bounded():
    text = "".join((ROOT / "csrc" / name).read_text() for name in ("prim.cuh", "tc_prim.cuh", "grouped_gemm_sm100.cu", "grouped_gemm_sm100_2cta.cu"))
    # each spin loop compares a timer against a limit
    for loop in re.findall(r"while \((?:!mbar_try|ld_acquire)[^{]*\{?[^}]*", text):
        assert "timeout_ns" in loop or "limit_ns" in loop, loop


def test_build_lists_existing_sources():
    for name in SOURCES:
        assert (source_dir() / name).exists(), name


def test_sm_budget_model():
    assert sms.theoretical_num_sms(148, 1, 256, 8, 810.0) == 148
    assert sms.theoretical_num_sms(148, 8, 256, 8, 0.0) == 148  # unknown NVLink -> all SMs
    n = sms.theoretical_num_sms(148, 8, 256, 8, 810.0)
    assert 16 <= n <= 148 and n % 4 == 0
    assert sms.theoretical_num_sms(148, 2, 64, 6, 810.0) <= 148
    p = sms.send_probability(8, 256, 8)
    assert abs(p - (1 - math.comb(224, 8) / math.comb(256, 8))) < 1e-12
    assert sms.nvlink_gbs(("a",)) == 0.0
    assert sms.nvlink_gbs(("no-such-gpu-1", "no-such-gpu-2")) == 0.0  # nvidia-smi missing or GPUs unknown


def test_nvtx_range_is_a_shared_noop_when_disabled():
    from nanoep_b200.utils import tracing

    if not tracing._ENABLED:
        assert tracing.nvtx_range("a") is tracing.nvtx_range("b")
    with tracing.nvtx_range("anything"):
        pass
