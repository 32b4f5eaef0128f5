"""Packaging: the CUDA/C++ sources travel inside the wheel (``nanoep_b200/_csrc``) and are compiled
for sm_100a on the target host with ``python -m nanoep_b200.utils.build`` (same arrangement as the
reference's setup.py:20-29, minus its JIT submodule)."""

import shutil
from pathlib import Path

from setuptools import setup
from setuptools.command.build_py import build_py

ROOT = Path(__file__).resolve().parent


class BuildWithSources(build_py):
    def run(self):
        super().run()
        target = Path(self.build_lib) / "nanoep_b200" / "_csrc"
        if target.exists():
            shutil.rmtree(target)
        shutil.copytree(ROOT / "csrc", target)


setup(cmdclass={"build_py": BuildWithSources})
