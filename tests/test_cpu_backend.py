"""Gloo world_size>1 tests of the pure-PyTorch backend (no GPU)."""

import pytest

from nanoep_b200.testing.spawn import run_gloo

from . import cpu_workers


def test_round_trip_identity_world2():
    assert run_gloo(2, cpu_workers.round_trip_identity) == [True, True]


@pytest.mark.parametrize("world,multiple", [(2, False), (2, True), (4, False)])
def test_all_kinds_against_oracle(world, multiple):
    assert all(run_gloo(world, cpu_workers.all_kinds, multiple, timeout=300))


@pytest.mark.parametrize("world", [2, 4])
def test_edge_geometries_against_oracle(world):
    assert run_gloo(world, cpu_workers.geometry_sweep, timeout=300) == [42] * world


def test_special_bit_patterns_are_moved_unchanged():
    assert all(run_gloo(2, cpu_workers.special_bits))


def test_argument_contract_and_lifetime():
    assert all(run_gloo(2, cpu_workers.misuse))


def test_config_mismatch_raises_everywhere():
    messages = run_gloo(2, cpu_workers.mismatched_config)
    assert messages[0] == messages[1] == "EPConfig mismatch across ranks"
