"""Multi-process tests over real CUDA IPC / NVLink: one process per GPU, launched with a hard timeout.

Needs >= 2 GPUs (skipped otherwise).  World sizes 2, 4 and 8 run when that many GPUs are visible.
"""

from pathlib import Path

import pytest
import torch

from nanoep_b200.testing.launcher import run_ranks

ROOT = Path(__file__).resolve().parent.parent
pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _gpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.parametrize("nproc", [2, 4, 8])
def test_public_api_worker(tmp_path, nproc):
    if _gpus() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    code, text = run_ranks(str(ROOT / "tests" / "gpu_worker.py"), nproc, log=tmp_path / "worker.log", cwd=ROOT, timeout=600, as_module=False)
    assert code == 0, text[-4000:]
    for rank in range(nproc):
        assert f"NANOEP_RANK_OK={rank} " in text, text[-4000:]


def test_example_moe_acceptance_profiles(tmp_path):
    """All delivery profiles of the forward MoE example (both layouts x four routing patterns, up to
    256 tokens x 7168 x top-8, async + cached) in one launch per world size."""
    from tests.acceptance_worker import PROFILES

    nproc = 2 if _gpus() < 4 else 4
    code, text = run_ranks(str(ROOT / "tests" / "acceptance_worker.py"), nproc, log=tmp_path / "accept.log", cwd=ROOT, timeout=600, as_module=False)
    assert code == 0, text[-4000:]
    for name in PROFILES:
        assert text.count(f"NANOEP_ACCEPT_OK={name} ") == nproc, (name, text[-4000:])


def test_example_moe_cli(tmp_path):
    nproc = 2 if _gpus() < 4 else 4
    code, text = run_ranks("nanoep_b200.examples.moe", nproc, args=["--async-op", "--cached"], log=tmp_path / "moe.log", cwd=ROOT, timeout=300)
    assert code == 0, text[-4000:]
    assert text.count("NANOEP_MOE_OK=") == nproc, text[-4000:]


@pytest.mark.parametrize("nproc", [2, 4])
def test_fused_moe_layer_multi(tmp_path, nproc):
    if _gpus() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    code, text = run_ranks(str(ROOT / "tests" / "moe_worker.py"), nproc, log=tmp_path / "moe_layer.log", cwd=ROOT, timeout=400, as_module=False)
    assert code == 0, text[-4000:]
    for rank in range(nproc):
        assert f"NANOEP_MOE_LAYER_OK={rank}" in text, text[-4000:]


def test_fused_moe_example(tmp_path):
    nproc = 2 if _gpus() < 4 else 4
    code, text = run_ranks("nanoep_b200.examples.fused_moe", nproc, log=tmp_path / "fused.log", cwd=ROOT, timeout=300)
    assert code == 0, text[-4000:]
    assert text.count("NANOEP_FUSED_MOE_OK=") == nproc, text[-4000:]
