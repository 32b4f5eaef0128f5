"""Fused MoE layer on one GPU (one rank, all experts local): dispatch -> tcgen05 SwiGLU GEMM ->
down GEMM with scatter epilogue -> reduce, against a PyTorch fp32 reference."""

from pathlib import Path

import pytest

from nanoep_b200.testing.launcher import run_ranks

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu


def test_fused_moe_layer_single_gpu(tmp_path):
    code, text = run_ranks(str(ROOT / "tests" / "moe_worker.py"), 1, log=tmp_path / "moe_layer.log", cwd=ROOT, timeout=300, as_module=False)
    assert code == 0, text[-4000:]
    assert "NANOEP_MOE_LAYER_OK=0" in text, text[-4000:]
