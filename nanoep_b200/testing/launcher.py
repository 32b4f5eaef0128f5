"""Bounded child-process launchers for multi-rank tests.

``run_logged`` runs a command in its own session with a hard timeout and kills the whole process
group on expiry so no GPU stays held (same contract as the reference's
nano_ep/testing/launcher.py:8-24).  ``run_ranks`` starts N ranks of a module through
``torch.distributed.run`` on 127.0.0.1 and returns the log text.
"""

from __future__ import annotations

import os
import signal
import socket
import subprocess
import sys
from pathlib import Path


def run_logged(command, *, log: Path, cwd, env=None, timeout: float = 300) -> int:
    # NANOEP_LOG_DIR keeps the workers' logs in one place after the test's temporary directory is gone
    # (the reference has NANO_EP_LOG_DIR for the same purpose, docs/testing.md:26).
    keep = os.environ.get("NANOEP_LOG_DIR")
    if keep:
        log = Path(keep) / log.name
    log.parent.mkdir(parents=True, exist_ok=True)
    with log.open("w") as output:
        process = subprocess.Popen(command, cwd=cwd, env=env, stdout=output, stderr=subprocess.STDOUT, start_new_session=True)
        try:
            return process.wait(timeout=timeout)
        except subprocess.TimeoutExpired:
            os.killpg(process.pid, signal.SIGKILL)
            process.wait()
            raise


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_ranks(target: str, nproc: int, *, args=(), log: Path, cwd, timeout: float = 300, env=None, as_module: bool = True) -> tuple[int, str]:
    full_env = dict(os.environ if env is None else env)
    full_env.setdefault("OMP_NUM_THREADS", "1")
    full_env["PYTHONPATH"] = os.pathsep.join([str(cwd)] + ([full_env["PYTHONPATH"]] if full_env.get("PYTHONPATH") else []))
    # Child ranks keep NCCL's in-switch (NVLS) reductions off: a rank that exits while its memory is
    # bound to such a switch object can fault its peers.
    full_env.setdefault("NCCL_NVLS_ENABLE", "0")
    command = [
        sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
        "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
    ]
    command += (["-m", target] if as_module else [target]) + list(args)
    code = run_logged(command, log=log, cwd=cwd, env=full_env, timeout=timeout)
    keep = os.environ.get("NANOEP_LOG_DIR")
    return code, (Path(keep) / log.name if keep else log).read_text()
