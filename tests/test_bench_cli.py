"""bench.py contract checks that need no GPU."""

import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_reference_arm_reports_unavailable():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1"],
                         capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "DeepJIT" in line["unavailable"]


def test_defaults_are_single_gpu_and_short():
    sys.path.insert(0, str(ROOT))
    import bench

    argv, sys.argv = sys.argv, ["bench.py"]
    try:
        args = bench.parse_args()
    finally:
        sys.argv = argv
    assert args.gpus == 1 and args.steps <= 50 and args.warmup >= 3
    assert (args.tokens, args.hidden, args.experts, args.topk) == (4096, 7168, 256, 8)


def test_clock_sampler_keeps_only_samples_inside_the_timed_windows(monkeypatch):
    sys.path.insert(0, str(ROOT))
    import bench

    class NoChild:
        def __init__(self, *a, **k):
            raise OSError("no child processes in this test")

    monkeypatch.setattr(bench.subprocess, "Popen", NoChild)
    sampler = bench.ClockSampler(0, "GPU-00000000")
    assert sampler.wait_ready(0.05) is False  # no child: gives up at once, never blocks a run
    sampler.windows = [[100.0, 101.0], [105.0, 106.0]]
    with open(sampler._path, "w") as f:
        f.write("source nvml\n")
        f.write("99.5 1200 1965 -\n")                      # before the first window
        f.write("100.5 1900 1965 sw_power_cap\n")
        f.write("103.0 300 1965 hw_slowdown\n")            # between the windows: not under load, ignored
        f.write("105.5 1950 1965 -\n")
        f.write("garbage line\n")
    got = sampler.summary()
    assert got["samples"] == 2 and got["sm_mhz"] == 1925.0 and got["sm_max_mhz"] == 1965.0
    assert got["reasons"] == ["sw_power_cap"] and got["source"] == "nvml" and got["window"] == "timed regions"
    assert not Path(sampler._path).exists()


def test_clock_records_of_all_ranks_are_merged_pessimistically():
    sys.path.insert(0, str(ROOT))
    import bench

    a = {"sm_mhz": 1950.0, "sm_max_mhz": 1965.0, "reasons": [], "samples": 5, "source": "nvml", "window": "timed regions"}
    b = {"sm_mhz": 1400.0, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"], "samples": 4, "source": "nvml", "window": "timed regions"}
    c = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "source": None, "window": "timed regions"}
    got = bench.merge_clock_summaries([a, b, c])
    assert got["sm_mhz"] == 1400.0 and got["sm_max_mhz"] == 1965.0 and got["reasons"] == ["sw_power_cap"] and got["samples"] == 9
    assert got["per_rank_sm_mhz"] == [1950.0, 1400.0, None]
    assert bench.merge_clock_summaries([c])["sm_mhz"] is None
