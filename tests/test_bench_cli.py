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
