"""The forward MoE example on the Gloo/CPU backend (2 ranks, no GPU)."""

from pathlib import Path

import pytest

from nanoep_b200.testing.launcher import run_ranks

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("extra", [["--layout", "expanded", "--cached"], ["--layout", "compact", "--pattern", "uneven", "--async-op"]])
def test_example_moe_cpu(tmp_path, extra):
    code, text = run_ranks(
        "nanoep_b200.examples.moe", 2, args=["--backend", "cpu", "--tokens", "17", "--hidden", "64", "--iterations", "2", *extra],
        log=tmp_path / "moe.log", cwd=ROOT, timeout=240,
    )
    assert code == 0, text[-3000:]
    assert text.count("NANOEP_MOE_OK=") == 2, text[-3000:]
