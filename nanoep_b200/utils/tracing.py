"""Optional NVTX ranges around the public operations (``NANOEP_NVTX=1``) and per-phase device timing.

The reference has no tracing beyond ``-lineinfo``.  Two facilities here:

* ``nvtx_range(name)``: a context manager that pushes an NVTX range when ``NANOEP_NVTX=1`` so a
  timeline profiler shows dispatch / combine / fused-layer steps; free when the variable is unset.
* ``phase_timing()``: a context manager that switches on the native per-kernel CUDA-event marks and
  yields a function returning ``{phase: [microseconds, ...]}`` for the operations issued inside.
"""

from __future__ import annotations

import contextlib
import os

_ENABLED = os.environ.get("NANOEP_NVTX") == "1"


class _NoRange:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NO_RANGE = _NoRange()


class _Range:
    def __init__(self, name):
        self.name = name

    def __enter__(self):
        import torch

        torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        import torch

        torch.cuda.nvtx.range_pop()
        return False


def nvtx_range(name: str):
    """Context manager: an NVTX range when ``NANOEP_NVTX=1``, otherwise a shared no-op object."""
    return _Range(name) if _ENABLED else _NO_RANGE


@contextlib.contextmanager
def phase_timing():
    from .build import load_extension

    ext = load_extension()
    ext.take_phase_timings()
    ext.set_phase_timing(True)
    collected: dict[str, list[float]] = {}

    def read():
        for name, us in ext.take_phase_timings():
            collected.setdefault(name, []).append(us)
        return collected

    try:
        yield read
    finally:
        ext.set_phase_timing(False)
        read()
