"""``CudaBuffer``: the public dispatch/combine object of the CUDA backend.

API surface and argument contract follow the reference's ``CudaBuffer``
(nano_ep/backends/cuda.py:89-444; docs/api.md): collective construction over a control group, fresh
and cached dispatch, combine, asynchronous completion events, idempotent collective close.

What differs underneath: receivers *pull* staged rows with bulk copies straight into the final
compact / expert-major tensors (no receive-side second pass), every remotely accessed window region
is double-buffered so each operation needs one peer barrier, and device-side failures surface as
Python exceptions from a status word instead of a device trap.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist
from torch.utils import deterministic

from ..config import EPConfig
from ..types import NativeCombineResult, NativeDispatchResult, NativeHandle, NativeLayout
from ..utils.sms import nvlink_gbs, theoretical_num_sms
from ..utils.tracing import nvtx_range
from . import bootstrap


def check_torch_deterministic():
    """Outputs are allocated uninitialised and fully written by kernels on another stream; filling
    them from the allocating stream would race (reference: nano_ep/backends/cuda.py:16-20)."""
    if torch.are_deterministic_algorithms_enabled() and deterministic.fill_uninitialized_memory:
        raise RuntimeError(
            "nanoep_b200 does not support deterministic algorithms together with fill_uninitialized_memory; "
            "disable one of these PyTorch settings"
        )


class CudaEvent:
    """Completion of an ``async_op`` call; keeps the operation's tensors alive until waited on."""

    def __init__(self, event, keepalive: tuple = ()):
        self.event = event
        self.keepalive = keepalive

    def current_stream_wait(self):
        """Make the current stream wait for the result and register the outputs with it."""
        self.event.current_stream_wait()

    def query(self) -> bool:
        return self.event.query()


class _OnDevice:
    """``torch.cuda.device(index)`` costs several microseconds per use; ranks normally sit on their device
    already, in which case this context manager does nothing."""

    def __init__(self, index: int):
        self.index = index
        self.inner = None

    def __enter__(self):
        if torch.cuda.current_device() != self.index:
            self.inner = torch.cuda.device(self.index)
            self.inner.__enter__()
        return self

    def __exit__(self, *exc):
        if self.inner is not None:
            self.inner.__exit__(*exc)
            self.inner = None
        return False


def _load_native():
    from ..utils.build import load_extension

    return load_extension()


def close_peer_window(window, group, device):
    """Drain the GPU, then unmap on every rank before any rank frees (two host barriers)."""
    torch.cuda.synchronize(device)
    dist.barrier(group=group)
    window.close_peer_mappings()
    dist.barrier(group=group)
    window.close()


class CudaBuffer:
    """Single-node expert-parallel buffer: one process per GPU, peers reached over NVLink."""

    HIDDEN_MULTIPLE = 256

    def __init__(
        self,
        group,
        config: EPConfig,
        *,
        allow_multiple_reduction: bool = False,
        wait_timeout_s: float | None = None,
        mailbox_timeout_s: float | None = None,
    ):
        # Limits of the bounded waits: device side (peer barrier, bulk copies) and host side (N/C mailbox).
        # Environment overrides: NANOEP_WAIT_TIMEOUT_S, NANOEP_MAILBOX_TIMEOUT_S.
        if wait_timeout_s is None:
            wait_timeout_s = float(os.environ.get("NANOEP_WAIT_TIMEOUT_S", "10"))
        if mailbox_timeout_s is None:
            mailbox_timeout_s = float(os.environ.get("NANOEP_MAILBOX_TIMEOUT_S", "60"))
        self._group = group
        self._config = config
        self._allow_multiple_reduction = allow_multiple_reduction
        self._world_size = dist.get_world_size(group=group)
        self._rank = dist.get_rank(group=group)
        self._window = None
        self._comm_stream = None
        self._closed = True
        self._auto_num_sms = None
        self._mailbox_timeout_s = float(mailbox_timeout_s)
        backend = dist.get_backend(group)
        if "gloo" not in str(backend):
            raise ValueError("CudaBuffer requires a Gloo control group")

        def probe():
            self._device = torch.cuda.current_device()
            props = torch.cuda.get_device_properties(self._device)
            self._device_sms = props.multi_processor_count
            return bootstrap.local_facts(config, allow_multiple_reduction, str(props.uuid))

        facts, errors = bootstrap.collective_step(group, "environment", probe)
        if errors:
            raise RuntimeError("CudaBuffer environment check failed: " + "; ".join(errors))
        bootstrap.validate_group_facts(facts, self._world_size, require_distinct_gpus=True, hidden_multiple=self.HIDDEN_MULTIPLE)
        self._gpu_uuids = tuple(f["gpu_uuid"] for f in facts)

        def allocate():
            self._backend = _load_native()
            self._window = self._backend.PeerWindow(
                self._rank,
                self._world_size,
                config.num_max_tokens_per_rank,
                config.hidden,
                config.num_topk,
                config.num_experts,
                float(wait_timeout_s),
                bool(allow_multiple_reduction),
            )
            self._layout = self._window.layout()
            return self._window.export_handle()

        handles, errors = bootstrap.collective_step(group, "allocation/export", allocate)
        stage = "allocation/export"
        if not errors:

            def connect():
                # each peer's GPU as this process sees it (by UUID; -1 when it is outside the visible set)
                visible = {str(torch.cuda.get_device_properties(i).uuid): i for i in range(torch.cuda.device_count())}
                self._window.import_handles(handles, [visible.get(uuid, -1) for uuid in self._gpu_uuids])
                self._comm_stream = torch.cuda.Stream(device=self._device)

            _, errors = bootstrap.collective_step(group, "import/stream", connect)
            stage = "import/stream"
        if errors:
            errors += self._rollback()
            self._comm_stream = None
            raise RuntimeError(f"CudaBuffer {stage} failed: " + "; ".join(errors))
        self._closed = False

    def _rollback(self) -> list[str]:
        """Collective unmap, then (only if every rank unmapped) collective free."""

        def unmap():
            if self._window is not None:
                torch.cuda.synchronize(self._device)
                self._window.close_peer_mappings()

        _, unmap_errors = bootstrap.collective_step(self._group, "unmap", unmap)
        if unmap_errors:
            return [e.replace(": ", " unmap: ", 1) for e in unmap_errors]

        def free():
            if self._window is not None:
                self._window.close()

        _, free_errors = bootstrap.collective_step(self._group, "free", free)
        return [e.replace(": ", " free: ", 1) for e in free_errors]

    # ------------------------------------------------------------------ properties
    @property
    def config(self) -> EPConfig:
        return self._config

    @property
    def rank(self) -> int:
        return self._rank

    @property
    def world_size(self) -> int:
        return self._world_size

    @property
    def allow_multiple_reduction(self) -> bool:
        return self._allow_multiple_reduction

    @property
    def comm_stream(self):
        return self._comm_stream

    @property
    def window(self):
        return self._window

    def _resolve_num_sms(self, num_sms: int | None, handle: NativeHandle | None) -> int:
        if num_sms is None:
            return self._device_sms if handle is None or handle.num_sms is None else handle.num_sms
        if isinstance(num_sms, bool) or not isinstance(num_sms, int) or not 0 <= num_sms <= self._device_sms:
            raise ValueError(f"num_sms must be an integer between 0 and {self._device_sms}")
        if num_sms > 0:
            return num_sms
        if self._auto_num_sms is None:
            self._auto_num_sms = theoretical_num_sms(
                self._device_sms, self._world_size, self._config.num_experts, self._config.num_topk, nvlink_gbs(self._gpu_uuids)
            )
        return self._auto_num_sms

    # ------------------------------------------------------------------ dispatch
    def dispatch(
        self,
        x: torch.Tensor,
        *,
        topk_idx: torch.Tensor | None = None,
        weights: torch.Tensor | None = None,
        handle: NativeHandle | None = None,
        do_expand: bool | None = None,
        alignment: int | None = None,
        zero_padding: bool = False,
        previous_event: torch.cuda.Event | None = None,
        async_op: bool = False,
        num_sms: int | None = None,
        tile_ready: torch.Tensor | None = None,
        ring_smem_limit: int = 0,
    ) -> NativeDispatchResult:
        """Send every token once to each rank that owns one of its experts; return exact layouts.

        ``tile_ready`` (optional, expert-major layout with zero padding only): a zeroed int32 tensor with
        one counter per 128 output rows; the pull kernel adds one per row once the row is in memory,
        so a consumer kernel on another stream can start on a row block as soon as it is complete.
        ``ring_smem_limit`` caps the pull kernel's shared-memory ring (bytes per CTA) so that such a
        consumer can share the SMs with it; 0 uses all of the CTA's shared memory.
        """
        check_torch_deterministic()
        if self._closed:
            raise RuntimeError("CudaBuffer is closed")
        expand, expert_alignment = resolve_layout_args(self, handle, topk_idx, do_expand, alignment)
        routing = handle.topk_idx if handle is not None else topk_idx
        if x.dim() != 2 or x.shape[1] != self._config.hidden:
            raise ValueError("x hidden dimension does not match the buffer configuration")
        if routing.shape != (x.shape[0], self._config.num_topk):
            raise ValueError("routing snapshot/topk_idx shape must match the buffer configuration")

        main_sms = self._resolve_num_sms(num_sms, handle)
        if handle is not None and handle.native_state is not None:
            with _OnDevice(self._device), nvtx_range("nanoep.dispatch.cached"):
                out_x, out_idx, out_w, completed = self._backend.dispatch_cached(
                    self._window, x, weights, handle.native_state, bool(zero_padding), main_sms, self._comm_stream.cuda_stream,
                    -1 if previous_event is None else previous_event.cuda_event, bool(async_op), self._mailbox_timeout_s,
                    tile_ready, int(ring_smem_limit),
                )
            event = CudaEvent(completed, keepalive=(self, x, routing, weights, handle)) if async_op else None
            return NativeDispatchResult(
                x=out_x, topk_idx=None if expand else out_idx, topk_weights=out_w if weights is not None else None, handle=handle, event=event
            )
        cached_metadata, cached_capacity = ([], 0) if handle is None else (handle_metadata(handle), handle.layout.expanded_capacity)
        with _OnDevice(self._device), nvtx_range("nanoep.dispatch.fresh" if handle is None else "nanoep.dispatch.cached"):
            outputs, metadata, counts, completed = self._backend.dispatch(
                [self._window],
                [x],
                [topk_idx],
                [weights],
                [cached_metadata],
                [cached_capacity],
                expert_alignment,
                expand,
                bool(zero_padding),
                main_sms,
                self._comm_stream.cuda_stream,
                -1 if previous_event is None else previous_event.cuda_event,
                bool(async_op),
                self._mailbox_timeout_s,
                [tile_ready],
                int(ring_smem_limit),
            )
        if handle is None:
            handle = build_handle(self, metadata[0], counts[0], expand, expert_alignment, x.dtype, main_sms)
            handle.native_state = self._backend.HandleState(list(metadata[0]), int(counts[0][1]), bool(expand))
        event = CudaEvent(completed, keepalive=(self, x, routing, weights, handle)) if async_op else None
        out = outputs[0]
        return NativeDispatchResult(
            x=out[0],
            topk_idx=None if expand else out[1],
            topk_weights=out[2] if weights is not None else None,
            handle=handle,
            event=event,
        )

    # ------------------------------------------------------------------ combine
    def combine(
        self,
        x: torch.Tensor,
        handle: NativeHandle,
        *,
        weights: torch.Tensor | None = None,
        bias: torch.Tensor | None = None,
        previous_event: torch.cuda.Event | None = None,
        async_op: bool = False,
        num_sms: int | None = None,
    ) -> NativeCombineResult:
        """Return expert outputs to their source tokens and sum them in FP32 (no gate weighting)."""
        check_torch_deterministic()
        if self._closed:
            raise RuntimeError("CudaBuffer is closed")
        if handle.owner is not self:
            raise ValueError("combine handle belongs to another CudaBuffer")
        if handle.config != self._config:
            raise ValueError("combine handle configuration does not match this CudaBuffer")
        validate_combine_inputs(self._config, handle, x, weights, bias, torch.device("cuda", self._device))
        main_sms = self._resolve_num_sms(num_sms, handle)
        if handle.native_state is not None:
            with _OnDevice(self._device), nvtx_range("nanoep.combine"):
                out_x, out_w, completed = self._backend.combine_single(
                    self._window, x, handle.native_state, weights, bias, self._allow_multiple_reduction, main_sms,
                    self._comm_stream.cuda_stream, -1 if previous_event is None else previous_event.cuda_event, bool(async_op),
                )
            event = CudaEvent(completed, keepalive=(self, x, handle, weights, bias)) if async_op else None
            return NativeCombineResult(x=out_x, topk_weights=out_w if weights is not None else None, event=event)
        with _OnDevice(self._device), nvtx_range("nanoep.combine"):
            outputs, completed = self._backend.combine(
                [self._window],
                [x],
                [handle_metadata(handle)],
                [handle.layout.expanded_capacity],
                [weights],
                [bias],
                handle.do_expand,
                self._allow_multiple_reduction,
                main_sms,
                self._comm_stream.cuda_stream,
                -1 if previous_event is None else previous_event.cuda_event,
                bool(async_op),
            )
        event = CudaEvent(completed, keepalive=(self, x, handle, weights, bias)) if async_op else None
        out = outputs[0]
        return NativeCombineResult(x=out[0], topk_weights=out[1] if weights is not None else None, event=event)

    # ------------------------------------------------------------------ misc
    def barrier(self):
        """Standalone peer barrier on the communication stream (shares the epoch sequence)."""
        if self._closed:
            raise RuntimeError("CudaBuffer is closed")
        self._window.barrier(self._comm_stream.cuda_stream)

    def check_status(self):
        """Raise if a kernel of this buffer reported an error (timeouts, bad routing, ...)."""
        self._window.check_status()

    def clear_status(self):
        """Forget a reported device status (after the application has dealt with it) so later calls run
        again.  Collective in spirit: a barrier timeout usually means the ranks' operation sequences have
        diverged, so clear it on every rank and re-synchronise (for example with ``barrier()``) first."""
        torch.cuda.synchronize(self._device)
        self._window.clear_status(self._comm_stream.cuda_stream)

    def close(self):
        """Collectively drain, unmap peers, then free.  Idempotent; never call from ``__del__``."""
        if self._closed:
            return
        close_peer_window(self._window, self._group, self._device)
        self._closed = True

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc_value, traceback):
        self.close()


# ---------------------------------------------------------------------- shared helpers
def resolve_layout_args(buffer, handle, topk_idx, do_expand, alignment) -> tuple[bool, int]:
    """Argument contract shared by every backend (reference: nano_ep/backends/cuda.py:264-284)."""
    if handle is not None:
        if handle.owner is not buffer:
            raise ValueError("cached handle belongs to another CudaBuffer")
        if topk_idx is not None:
            raise ValueError("cached dispatch uses the handle snapshot; omit topk_idx")
        if alignment is not None and alignment != handle.alignment:
            raise ValueError("cached dispatch must retain the handle alignment")
        if do_expand is not None and do_expand != handle.do_expand:
            raise ValueError("cached dispatch must retain the handle layout")
    elif topk_idx is None:
        raise ValueError("fresh dispatch requires topk_idx")
    if alignment is not None and (isinstance(alignment, bool) or not isinstance(alignment, int) or alignment <= 0):
        raise ValueError("alignment must be a positive integer")
    if do_expand is not None and not isinstance(do_expand, bool):
        raise ValueError("do_expand must be bool or None")
    if handle is not None:
        return handle.do_expand, handle.alignment
    return (False if do_expand is None else do_expand), (1 if alignment is None else alignment)


def handle_metadata(handle: NativeHandle) -> list[torch.Tensor]:
    layout = handle.layout
    return [
        layout.recv_metadata,
        layout.expert_counts,
        layout.expert_offsets,
        handle.dst_slots,
        handle.send_counts,
        handle.topk_idx,
        layout.recv_rank_prefix,
        handle.slot_map,
    ]


def build_handle(owner, metadata, counts, expand, alignment, x_dtype, num_sms) -> NativeHandle:
    recv_count, expanded_capacity = counts
    layout = NativeLayout(
        recv_metadata=metadata[0],
        expert_counts=metadata[1],
        expert_offsets=metadata[2],
        recv_rank_prefix=metadata[6],
        recv_count=int(recv_count),
        expanded_capacity=int(expanded_capacity),
    )
    return NativeHandle(
        config=owner.config,
        rank=owner.rank,
        world_size=owner.world_size,
        do_expand=expand,
        alignment=alignment,
        topk_idx=metadata[5],
        layout=layout,
        dst_slots=metadata[3],
        send_counts=metadata[4],
        owner=owner,
        x_dtype=x_dtype,
        num_sms=num_sms,
        slot_map=metadata[7],
    )


def validate_combine_inputs(config: EPConfig, handle: NativeHandle, x, weights, bias, device) -> None:
    layout = handle.layout
    rows = layout.expanded_capacity if handle.do_expand else layout.recv_count
    if x.device != device or x.dtype != torch.bfloat16 or x.shape != (rows, config.hidden) or not x.is_contiguous():
        raise ValueError("combine x must be contiguous bfloat16 on the buffer's device with the handle's exact receive shape")
    weight_shape = (rows,) if handle.do_expand else (rows, config.num_topk)
    if weights is not None and (
        weights.device != device or weights.dtype != torch.float32 or weights.shape != weight_shape or not weights.is_contiguous()
    ):
        raise ValueError("combine weights must be contiguous float32 on the buffer's device with the handle's receive layout")
    tokens = handle.topk_idx.shape[0]
    if bias is not None and (
        bias.device != device or bias.dtype != x.dtype or bias.shape != (tokens, config.hidden) or not bias.is_contiguous()
    ):
        raise ValueError("combine bias must be contiguous source [T,H], with the x dtype on this buffer's device")
