"""nanoep_b200: single-node expert-parallel dispatch and combine for PyTorch on B200 (sm_100a).

Public surface (same names as the reference package, nano_ep/__init__.py:3-16, plus the CPU backend,
the one-GPU logical group and the fused MoE layer)::

    from nanoep_b200 import EPConfig, CudaBuffer, CpuBuffer
"""

from .config import EPConfig
from .parallel.cpu_buffer import CpuBuffer, CpuEvent
from .parallel.cuda_buffer import CudaBuffer, CudaEvent
from .parallel.emulated import EmulatedGroup
from .types import NativeCombineResult, NativeDispatchResult, NativeHandle, NativeLayout

__version__ = "0.1.0"

__all__ = [
    "CpuBuffer",
    "CpuEvent",
    "CudaBuffer",
    "CudaEvent",
    "EPConfig",
    "EmulatedGroup",
    "NativeCombineResult",
    "NativeDispatchResult",
    "NativeHandle",
    "NativeLayout",
]
