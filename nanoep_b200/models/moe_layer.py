"""Expert-parallel SwiGLU MoE layer built on dispatch/combine and the tcgen05 grouped GEMM.

    y[t] = sum_k  w[t,k] * W2[e_k] @ ( silu(W1g[e_k] @ x[t]) * (W1u[e_k] @ x[t]) )

The reference library leaves the expert computation to the caller (its example uses element-wise
experts, nano_ep/examples/moe.py:19-40).  This layer is the fused path:

* dispatch runs with the expert-major layout, 128-row alignment and zero padding, with a small
  shared-memory ring per SM, and announces every finished row in per-block counters;
* the up/gate grouped GEMM (SwiGLU epilogue) starts at once on the SAME SMs (its operand pipeline is
  one stage shorter so both kernels fit in shared memory) and consumes row blocks as their counters
  fill, so the NVLink pull hides under tensor-core work;
* the down-projection GEMM applies the gate weight in FP32 in its epilogue, stages each bf16 output
  row in shared memory and bulk-stores it straight into the source rank's return partition over
  NVLink; a peer barrier and the source-side FP32 reduction finish the combine.

``fuse_combine=False`` / ``overlap_dispatch=False`` select the unfused compositions of the same
public operations (used as correctness and performance baselines).
"""

from __future__ import annotations

import torch

from ..ops import grouped_gemm as gg
from ..parallel.cuda_buffer import CudaBuffer, handle_metadata

ALIGNMENT = 128


class ExpertParallelMoE:
    def __init__(self, buffer: CudaBuffer, w13: torch.Tensor, w2: torch.Tensor, *, fuse_combine: bool = True,
                 overlap_dispatch: bool = False, comm_ring_bytes: int = 80 * 1024, cta_pairs: bool | None = None):
        cfg = buffer.config
        local = cfg.num_experts // buffer.world_size
        if w13.dim() != 3 or w13.shape[0] != local or w13.shape[2] != cfg.hidden or w13.shape[1] % 256:
            raise ValueError("w13 must be [local_experts, 2*I, hidden] with I a multiple of 128")
        inner = w13.shape[1] // 2
        if w2.shape != (local, cfg.hidden, inner):
            raise ValueError("w2 must be [local_experts, hidden, I]")
        if w13.dtype != torch.bfloat16 or w2.dtype != torch.bfloat16 or not (w13.is_contiguous() and w2.is_contiguous()):
            raise ValueError("expert weights must be contiguous bfloat16")
        if cfg.hidden % 256 or inner % 64:
            raise ValueError("hidden must be a multiple of 256 and I a multiple of 64")
        self.buffer, self.w13, self.w2 = buffer, w13, w2
        self.inner = inner
        # The scatter epilogue returns one row per choice; a buffer that pre-reduces per rank has no partitions for that.
        self.fuse_combine = fuse_combine and not buffer.allow_multiple_reduction
        self.overlap_dispatch = overlap_dispatch
        self.device = w13.device
        self.comm_ring_bytes = int(comm_ring_bytes)
        # tcgen05 cta_group::2 kernels (two SMs share each weight tile).  None = decide per call: a pair
        # needs two row blocks of the same expert, so with few blocks per expert the half-empty last
        # pairs cost more than the shared weight tiles save.
        self.cta_pairs = cta_pairs
        self.local_experts = local
        rows_cap = buffer.world_size * cfg.num_max_tokens_per_rank * min(cfg.num_topk, local) + local * (ALIGNMENT - 1)
        blocks = rows_cap // ALIGNMENT + 2
        self._tile_ready = torch.zeros(blocks, dtype=torch.int32, device=self.device)
        self._tile_expected = torch.full((blocks,), ALIGNMENT, dtype=torch.int32, device=self.device)
        self._ext = gg._ext()
        self.serialize_overlap = False  # diagnostics: run the overlap-mode kernels back to back instead of concurrently
        self.profile = False  # when set, forward() records CUDA events between its steps (see last_profile)
        self.last_profile: dict[str, float] = {}

    def forward(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor, *, handle=None, bias=None) -> torch.Tensor:
        buf = self.buffer
        stream = torch.cuda.current_stream(self.device)
        overlap = self.overlap_dispatch
        marks = []

        def mark(name):
            if self.profile:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record(stream)
                marks.append((name, ev))

        mark("start")
        if overlap:
            self._tile_ready.zero_()
        got = buf.dispatch(
            x, topk_idx=None if handle is not None else topk_idx, weights=topk_weights, handle=handle,
            do_expand=True if handle is None else None, alignment=ALIGNMENT if handle is None else None, zero_padding=True,
            async_op=overlap, tile_ready=self._tile_ready if overlap else None,
            ring_smem_limit=self.comm_ring_bytes if overlap else 0,
        )
        h_in, offsets = got.x, got.handle.layout.expert_offsets
        pairs = self.cta_pairs
        if pairs is None:
            pairs = got.handle.layout.expanded_capacity >= 6 * ALIGNMENT * self.local_experts
        if overlap:
            # The GEMM must not wait for the whole dispatch: it is gated per row block by the counters.
            h_in.record_stream(stream)
            if self.serialize_overlap:
                got.event.current_stream_wait()
                mark("dispatch_small_ring")
            h = gg.grouped_gemm(h_in, self.w13, offsets, swiglu=True, tile_ready=self._tile_ready, tile_expected=self._tile_expected,
                                stages=3, pair=pairs)
            got.event.current_stream_wait()  # metadata and slot weights are complete from here on
            mark("dispatch+up_gemm")
        else:
            mark("dispatch")
            h = gg.grouped_gemm(h_in, self.w13, offsets, swiglu=True, pair=pairs)
            mark("up_gemm")
        self.last_handle = got.handle
        if self.fuse_combine:
            window = buf.window
            self._ext.grouped_gemm_scatter(window, h, self.w2, offsets, got.handle.slot_map, got.handle.layout.recv_metadata,
                                           got.topk_weights, gg.status_tensor(self.device), 0, 5.0, pairs)
            mark("down_gemm_scatter")
            out = self._ext.combine_finish([window], [handle_metadata(got.handle)], [bias])[0]
            mark("barrier+reduce")
            self._collect(marks)
            return out
        y = gg.grouped_gemm(h, self.w2, offsets, row_scale=got.topk_weights, pair=pairs)  # gate weight in FP32 in the epilogue
        mark("down_gemm")
        out = buf.combine(y, got.handle, bias=bias).x
        mark("combine")
        self._collect(marks)
        return out

    def _collect(self, marks):
        if not self.profile or not marks:
            return
        marks[-1][1].synchronize()
        self.last_profile = {marks[i][0]: marks[i - 1][1].elapsed_time(marks[i][1]) * 1e3 for i in range(1, len(marks))}

    __call__ = forward


def dense_reference(x, topk_idx, topk_weights, w13_all, w2_all) -> torch.Tensor:
    """fp32 PyTorch reference with the layer's rounding points (bf16 after SwiGLU and per assignment)."""
    T, K = topk_idx.shape
    inner = w13_all.shape[1] // 2
    out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
    for k in range(K):
        for e in topk_idx[:, k].unique().tolist():
            if e < 0:
                continue
            rows = (topk_idx[:, k] == e).nonzero().flatten()
            gu = x[rows].float() @ w13_all[e].float().t()
            h = (torch.nn.functional.silu(gu[:, :inner]) * gu[:, inner:]).to(torch.bfloat16)
            y = (h.float() @ w2_all[e].float().t()) * topk_weights[rows, k, None].float()
            out[rows] += y.to(torch.bfloat16).float()
    return out.to(torch.bfloat16)
