"""The round-trip check that ``bench.py`` prints as ``"verified"`` must pass on a correct backend and must notice a
wrong one.  Runs the check itself on two Gloo ranks over the CPU backend (no GPU)."""

import sys
from pathlib import Path
from types import SimpleNamespace

import pytest

from nanoep_b200.testing.spawn import run_gloo

ROOT = Path(__file__).resolve().parent.parent


class _Tampering:
    """A buffer whose combine flips one bit of one element on one rank."""

    def __init__(self, inner, rank, what):
        self._inner, self._rank, self._what = inner, rank, what

    def dispatch(self, *a, **k):
        got = self._inner.dispatch(*a, **k)
        if self._what == "dispatch" and self._rank == 1 and got.x.numel():
            slots = got.handle.layout.recv_metadata[:, 2:]
            got.x.view(__import__("torch").int16)[int(slots[slots >= 0][0]), 0] ^= 1  # a row that holds a token, not padding
        return got

    def combine(self, *a, **k):
        back = self._inner.combine(*a, **k)
        if self._what == "combine" and self._rank == 1:
            back.x.view(__import__("torch").int16)[3, 5] ^= 1
        return back


def _check(rank, world, expand, multiple, tamper):
    import torch
    import torch.distributed as dist

    sys.path.insert(0, str(ROOT))
    import bench
    from nanoep_b200 import CpuBuffer, EPConfig
    from nanoep_b200.testing.cases import balanced_routing

    args = SimpleNamespace(experts=8, topk=3, hidden=64, tokens=19, alignment=4, num_sms=None, multiple_reduction=multiple)
    x = torch.randn(args.tokens, args.hidden, generator=torch.Generator().manual_seed(rank)).to(torch.bfloat16)
    idx, w = balanced_routing(args.tokens, args.experts, args.topk, seed=7 + rank)
    with CpuBuffer(dist.group.WORLD, EPConfig(args.experts, args.topk, args.hidden, args.tokens), allow_multiple_reduction=multiple) as inner:
        buf = _Tampering(inner, rank, tamper) if tamper else inner
        ok, note = bench.verify_round_trip(args, buf, rank, world, torch.device("cpu"), dist.group.WORLD, x, idx, w, expand)
    return ok, note


@pytest.mark.parametrize("expand,multiple", [(True, False), (True, True), (False, False)])
def test_check_passes_on_a_correct_backend(expand, multiple):
    for ok, note in run_gloo(2, _check, expand, multiple, None):
        assert ok, note
        assert "bit for bit" in note


@pytest.mark.parametrize("tamper,needle", [("combine", "round trip differs"), ("dispatch", "differs from its source token")])
def test_check_notices_a_single_flipped_bit(tamper, needle):
    results = run_gloo(2, _check, True, False, tamper)
    # every rank reports the same verdict, and it names the rank and the kind of mismatch
    assert all(not ok for ok, _ in results)
    assert all("rank 1" in note and needle in note for _, note in results), results
