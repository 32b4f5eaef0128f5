"""ctypes access to the allocation-free receive-planning entry point (csrc/noalloc).

For callers that may not allocate device memory when they need a receive plan (see the header for
who they are).  The function below only forwards pointers; the native call allocates nothing.
"""

from __future__ import annotations

import ctypes
import functools

MAX_LOCAL_EXPERTS = 4096
OK, TOO_LARGE, BAD_ARGUMENT, CUDA_ERROR = 0, 1, 2, 3


@functools.cache
def library() -> ctypes.CDLL:
    from ..utils.build import build_noalloc

    lib = ctypes.CDLL(str(build_noalloc()))
    lib.nep_plan_rows_noalloc.restype = ctypes.c_int
    lib.nep_plan_rows_noalloc.argtypes = [
        ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
        ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
    ]
    lib.nep_noalloc_last_error.restype = ctypes.c_char_p
    return lib


def plan_rows_noalloc(topk_i32, source_rank, expert_lo, local_experts, expert_offsets_i32, expand, meta_out, row_count_out, stream=None) -> int:
    """Enqueue the plan on ``stream`` (default: torch's current stream); returns the native status code.

    All tensors are caller-owned int32 CUDA tensors; nothing is allocated here or in the native call.
    """
    import torch

    if stream is None:
        stream = torch.cuda.current_stream().cuda_stream
    offsets_ptr = None if expert_offsets_i32 is None else expert_offsets_i32.data_ptr()
    return library().nep_plan_rows_noalloc(
        topk_i32.data_ptr(), topk_i32.shape[0], topk_i32.shape[1], source_rank, expert_lo, local_experts,
        offsets_ptr, int(bool(expand)), meta_out.data_ptr(), row_count_out.data_ptr(), stream,
    )
