"""The sdist/wheel carry every native source and the installed package finds them (no compile, no GPU)."""

import subprocess
import sys
from pathlib import Path


def test_wheel_bundles_native_sources_and_imports():
    root = Path(__file__).resolve().parent.parent
    done = subprocess.run([sys.executable, "-m", "nanoep_b200.utils.check_package"], cwd=root, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-2000:]
    assert done.stdout.strip().endswith("package ok")
