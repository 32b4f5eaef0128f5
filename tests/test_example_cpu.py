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


def test_acceptance_profiles_cpu(tmp_path):
    """The acceptance worker itself (all profiles that are small enough for the CPU backend), 2 Gloo ranks."""
    from tests.acceptance_worker import PROFILES

    small = [n for n in PROFILES if not n.startswith("wide-")]
    code, text = run_ranks(
        str(ROOT / "tests" / "acceptance_worker.py"), 2, log=tmp_path / "accept.log", cwd=ROOT, timeout=600, as_module=False,
        env={**__import__("os").environ, "NANOEP_ACCEPT_BACKEND": "cpu", "NANOEP_ACCEPT_PROFILES": ",".join(small)},
    )
    assert code == 0, text[-3000:]
    for name in small:
        assert text.count(f"NANOEP_ACCEPT_OK={name} ") == 2, (name, text[-3000:])
