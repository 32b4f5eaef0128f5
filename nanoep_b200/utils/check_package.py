"""Build an sdist and a wheel, check that every native source is bundled, and import the wheel
from outside the checkout (``--compile`` also builds the extension there; needs nvcc).

    python -m nanoep_b200.utils.check_package [--compile]

Counterpart of the reference's tools/check_package.py:13-76.
"""

from __future__ import annotations

import argparse
import shutil
import subprocess
import sys
import tempfile
import zipfile
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent.parent


def main():
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--compile", action="store_true")
    args = parser.parse_args()
    with tempfile.TemporaryDirectory() as tmp:
        tmp = Path(tmp)
        # build from a copy so that no build/ or egg-info directory appears in the checkout
        src = tmp / "src"
        src.mkdir()
        for name in ("pyproject.toml", "setup.py", "MANIFEST.in", "README.md"):
            shutil.copy(ROOT / name, src / name)
        shutil.copytree(ROOT / "csrc", src / "csrc")
        shutil.copytree(ROOT / "nanoep_b200", src / "nanoep_b200", ignore=shutil.ignore_patterns("_ext", "_csrc", "__pycache__"))
        subprocess.run([sys.executable, "-m", "pip", "wheel", "--no-deps", "--no-build-isolation", "-w", str(tmp / "dist"), str(src)], check=True)
        wheel = next((tmp / "dist").glob("nanoep_b200-*.whl"))
        names = set(zipfile.ZipFile(wheel).namelist())
        for src in (ROOT / "csrc").rglob("*"):
            if src.is_file():
                rel = "nanoep_b200/_csrc/" + str(src.relative_to(ROOT / "csrc"))
                assert rel in names, f"{rel} missing from the wheel"
        site = tmp / "site"
        subprocess.run([sys.executable, "-m", "pip", "install", "--no-deps", "--target", str(site), str(wheel)], check=True)
        probe = "import nanoep_b200, nanoep_b200.utils.build as b; print(b.source_dir())"
        if args.compile:
            probe += "; b.build_all()"
        out = subprocess.run([sys.executable, "-c", probe], cwd=tmp, env={"PYTHONPATH": str(site), "PATH": "/usr/local/cuda/bin:/usr/bin:/bin"},
                             check=True, capture_output=True, text=True).stdout
        assert "_csrc" in out, out
    print("package ok")


if __name__ == "__main__":
    main()
