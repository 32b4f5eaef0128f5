"""A whole expert-parallel group on ONE GPU ("logical peers").

Each logical rank owns a separate peer window in the same process; the windows adopt one another as
peers and every phase of dispatch/combine runs as a single multi-rank launch (grid.y = rank), so the
cross-rank waits inside the kernels are satisfied within one launch.  This exercises all addressing,
counting and protocol logic without NVLink; real peer traffic needs one process per GPU
(``CudaBuffer``).  The reference tests the same thing with hand-built probe kernels
(tests/native/test_peer_runtime.py:235-348, tests/native/combine_probe.cu).
"""

from __future__ import annotations

import torch

from ..config import EPConfig
from ..types import NativeCombineResult, NativeDispatchResult, NativeHandle
from .cuda_buffer import _load_native, build_handle, check_torch_deterministic, handle_metadata, resolve_layout_args, validate_combine_inputs


class _RankView:
    """What a handle's ``owner`` points to for one logical rank."""

    def __init__(self, group: "EmulatedGroup", rank: int):
        self.group = group
        self.rank = rank
        self.config = group.config
        self.world_size = group.world_size


class EmulatedGroup:
    def __init__(self, world_size: int, config: EPConfig, *, allow_multiple_reduction: bool = False, device=None, wait_timeout_s: float = 5.0):
        if world_size < 1 or world_size > 32 or world_size & (world_size - 1):
            raise ValueError("world size must be a power of two in [1, 32]")
        if config.num_experts % world_size:
            raise ValueError("num_experts must be divisible by world_size")
        if config.hidden % 256:
            raise ValueError("hidden must be a multiple of 256 (the kernels move rows in whole 32-lane passes of 16-byte chunks)")
        self.config = config
        self.world_size = world_size
        self.allow_multiple_reduction = allow_multiple_reduction
        self.device = torch.cuda.current_device() if device is None else device
        self._backend = _load_native()
        with torch.cuda.device(self.device):
            self.windows = [
                self._backend.PeerWindow(
                    r, world_size, config.num_max_tokens_per_rank, config.hidden, config.num_topk, config.num_experts, float(wait_timeout_s),
                    bool(allow_multiple_reduction),
                )
                for r in range(world_size)
            ]
            for w in self.windows:
                w.adopt_peers(self.windows)
            self.comm_stream = torch.cuda.Stream(device=self.device)
            self.device_sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.views = [_RankView(self, r) for r in range(world_size)]
        self._closed = False

    def _sms(self, num_sms):
        if num_sms is None:
            return max(1, self.device_sms // self.world_size)
        return num_sms

    def dispatch(
        self,
        xs,
        *,
        topk_idx=None,
        weights=None,
        handles=None,
        do_expand=None,
        alignment=None,
        zero_padding=False,
        async_op=False,
        num_sms=None,
    ) -> list[NativeDispatchResult]:
        check_torch_deterministic()
        if self._closed:
            raise RuntimeError("EmulatedGroup is closed")
        R = self.world_size
        topk_idx = topk_idx if topk_idx is not None else [None] * R
        weights = weights if weights is not None else [None] * R
        handles = handles if handles is not None else [None] * R
        expand, align = resolve_layout_args(self.views[0], handles[0], topk_idx[0], do_expand, alignment)
        for r in range(1, R):
            assert resolve_layout_args(self.views[r], handles[r], topk_idx[r], do_expand, alignment) == (expand, align)
        cached = [[] if h is None else handle_metadata(h) for h in handles]
        capacity = [0 if h is None else h.layout.expanded_capacity for h in handles]
        with torch.cuda.device(self.device):
            outputs, metadata, counts, completed = self._backend.dispatch(
                self.windows, list(xs), list(topk_idx), list(weights), cached, capacity, align, expand, bool(zero_padding),
                self._sms(num_sms), self.comm_stream.cuda_stream, -1, bool(async_op), 30.0,
            )
        results = []
        for r in range(R):
            handle = handles[r]
            if handle is None:
                handle = build_handle(self.views[r], metadata[r], counts[r], expand, align, xs[r].dtype, self._sms(num_sms))
            out = outputs[r]
            results.append(
                NativeDispatchResult(
                    x=out[0],
                    topk_idx=None if expand else out[1],
                    topk_weights=out[2] if weights[r] is not None else None,
                    handle=handle,
                    event=completed,
                )
            )
        return results

    def combine(self, xs, handles: list[NativeHandle], *, weights=None, bias=None, async_op=False, num_sms=None) -> list[NativeCombineResult]:
        check_torch_deterministic()
        if self._closed:
            raise RuntimeError("EmulatedGroup is closed")
        R = self.world_size
        weights = weights if weights is not None else [None] * R
        bias = bias if bias is not None else [None] * R
        dev = torch.device("cuda", self.device)
        for r in range(R):
            if handles[r].owner is not self.views[r]:
                raise ValueError("combine handle belongs to another buffer")
            validate_combine_inputs(self.config, handles[r], xs[r], weights[r], bias[r], dev)
        with torch.cuda.device(self.device):
            outputs, completed = self._backend.combine(
                self.windows, list(xs), [handle_metadata(h) for h in handles], [h.layout.expanded_capacity for h in handles],
                list(weights), list(bias), handles[0].do_expand, self.allow_multiple_reduction, self._sms(num_sms),
                self.comm_stream.cuda_stream, -1, bool(async_op),
            )
        return [
            NativeCombineResult(x=outputs[r][0], topk_weights=outputs[r][1] if weights[r] is not None else None, event=completed)
            for r in range(R)
        ]

    def barrier(self):
        self._backend.group_barrier(self.windows, self.comm_stream.cuda_stream)

    def check_status(self):
        for w in self.windows:
            w.check_status()

    def close(self):
        if self._closed:
            return
        torch.cuda.synchronize(self.device)
        for w in self.windows:
            w.close_peer_mappings()
        for w in self.windows:
            w.close()
        self._closed = True

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
