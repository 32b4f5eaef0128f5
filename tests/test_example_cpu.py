"""The forward MoE example on the Gloo/CPU backend (2 ranks, no GPU)."""

from pathlib import Path

import pytest

from nanoep_b200.testing.launcher import run_ranks

ROOT = Path(__file__).resolve().parent.parent


PROFILES = [
    ["--layout", "expanded", "--cached"],
    ["--layout", "compact", "--pattern", "uneven", "--async-op"],
    ["--layout", "expanded", "--pattern", "masked", "--multiple-reduction", "--alignment", "4"],
    ["--layout", "compact", "--pattern", "skew", "--cached", "--async-op", "--topk", "4", "--experts-per-rank", "3"],
]


@pytest.mark.parametrize("extra", PROFILES)
def test_example_moe_cpu(tmp_path, extra):
    code, text = run_ranks(
        "nanoep_b200.examples.moe", 2, args=["--backend", "cpu", "--tokens", "17", "--hidden", "64", "--iterations", "2", *extra],
        log=tmp_path / "moe.log", cwd=ROOT, timeout=240,
    )
    assert code == 0, text[-3000:]
    assert text.count("NANOEP_MOE_OK=") == 2, text[-3000:]
