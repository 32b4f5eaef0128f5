"""Pure-PyTorch CPU backend over a Gloo group.

Implements the same public API as ``CudaBuffer`` with ordinary tensor ops and object collectives, so
the whole dispatch -> experts -> combine round trip can run without a GPU.  The reference ships no
CPU backend (its export strips the simulator, tools/check_package.py:41,68); the behaviour here is
derived from the documented semantics (docs/api.md) and serves as the portable fallback and as a
second, independent implementation to compare the CUDA kernels against.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..config import EPConfig
from ..types import NativeCombineResult, NativeDispatchResult, NativeHandle, NativeLayout
from . import bootstrap
from .cuda_buffer import resolve_layout_args, validate_combine_inputs


class CpuEvent:
    """Completion object of the CPU backend: everything is already complete."""

    def current_stream_wait(self):
        return None

    def query(self) -> bool:
        return True


def receive_layout(all_topk: list[torch.Tensor], rank: int, local_experts: int, alignment: int, expand: bool):
    """Vectorised receive plan of ``rank``: rows ordered by (source rank, token)."""
    lo = rank * local_experts
    topk = all_topk[0].shape[1]
    src_ranks, src_tokens, local_rows = [], [], []
    for src, idx in enumerate(all_topk):
        local = torch.where((idx >= lo) & (idx < lo + local_experts), idx - lo, torch.full_like(idx, -1))
        keep = (local >= 0).any(dim=1)
        tokens = keep.nonzero().flatten()
        src_ranks.append(torch.full_like(tokens, src))
        src_tokens.append(tokens)
        local_rows.append(local[tokens])
    src_ranks = torch.cat(src_ranks)
    src_tokens = torch.cat(src_tokens)
    local = torch.cat(local_rows).reshape(-1, topk)
    flat = local.flatten()
    valid = flat >= 0
    counts = torch.bincount(flat[valid], minlength=local_experts).to(torch.int64)
    padded = (counts + alignment - 1) // alignment * alignment
    offsets = torch.cat([torch.zeros(1, dtype=torch.int64), padded.cumsum(0)])
    slots = torch.full_like(flat, -1)
    if valid.any():
        # rank of each assignment among the assignments of the same expert, in row-major order
        order = torch.argsort(flat[valid], stable=True)
        sorted_experts = flat[valid][order]
        starts = torch.cat([torch.zeros(1, dtype=torch.int64), counts.cumsum(0)])[sorted_experts]
        within = torch.arange(len(order)) - starts
        assigned = torch.empty_like(within)
        assigned[order] = offsets[sorted_experts] + within
        slots[valid] = assigned
    slots = slots.reshape(-1, topk)
    prefix = torch.bincount(src_ranks, minlength=len(all_topk)).cumsum(0).to(torch.int64)
    meta_tail = slots if expand else local
    recv_metadata = torch.cat([src_ranks[:, None], src_tokens[:, None], meta_tail], dim=1).to(torch.int32)
    return recv_metadata, local, slots, counts, offsets, prefix


class CpuBuffer:
    HIDDEN_MULTIPLE = 1

    def __init__(self, group, config: EPConfig, *, allow_multiple_reduction: bool = False):
        self._group = group
        self._config = config
        self._allow_multiple_reduction = allow_multiple_reduction
        self._world_size = dist.get_world_size(group=group)
        self._rank = dist.get_rank(group=group)
        self._closed = True
        facts, errors = bootstrap.collective_step(
            group, "environment", lambda: bootstrap.local_facts(config, allow_multiple_reduction, None)
        )
        if errors:
            raise RuntimeError("CpuBuffer environment check failed: " + "; ".join(errors))
        bootstrap.validate_group_facts(facts, self._world_size, require_distinct_gpus=False, hidden_multiple=self.HIDDEN_MULTIPLE)
        self._local_experts = config.num_experts // self._world_size
        self._closed = False

    config = property(lambda self: self._config)
    rank = property(lambda self: self._rank)
    world_size = property(lambda self: self._world_size)

    def _check_payload(self, x, topk_idx, weights):
        cfg = self._config
        if x.device.type != "cpu" or x.dtype != torch.bfloat16 or x.dim() != 2 or x.shape[1] != cfg.hidden or not x.is_contiguous():
            raise ValueError("x must be a contiguous CPU bfloat16 [T, hidden] tensor")
        if x.shape[0] > cfg.num_max_tokens_per_rank:
            raise ValueError("x has more tokens than num_max_tokens_per_rank")
        if topk_idx is not None:
            if topk_idx.dtype != torch.int64 or topk_idx.shape != (x.shape[0], cfg.num_topk):
                raise ValueError("topk_idx must be int64 [T, num_topk]")
            if ((topk_idx < -1) | (topk_idx >= cfg.num_experts)).any():
                raise ValueError("topk_idx holds an expert id outside [-1, num_experts)")
        if weights is not None and (weights.dtype != torch.float32 or weights.shape != (x.shape[0], cfg.num_topk)):
            raise ValueError("weights must be float32 [T, num_topk]")

    def dispatch(
        self, x, *, topk_idx=None, weights=None, handle=None, do_expand=None, alignment=None, zero_padding=False,
        previous_event=None, async_op=False, num_sms=None,
    ) -> NativeDispatchResult:
        if self._closed:
            raise RuntimeError("CpuBuffer is closed")
        expand, align = resolve_layout_args(self, handle, topk_idx, do_expand, alignment)
        self._check_payload(x, topk_idx, weights)
        routing = handle.topk_idx if handle is not None else topk_idx.clone()
        if routing.shape[0] != x.shape[0]:
            raise ValueError("routing snapshot/topk_idx shape must match x")
        gathered = bootstrap.gather_objects(self._group, {"x": x, "topk": routing, "w": weights})
        all_topk = [g["topk"] for g in gathered]
        if handle is None:
            meta, local, slots, counts, offsets, prefix = receive_layout(all_topk, self._rank, self._local_experts, align, expand)
            in_rank = torch.zeros((x.shape[0], self._world_size), dtype=torch.bool)
            valid = routing >= 0
            owner = torch.where(valid, routing // self._local_experts, torch.zeros_like(routing))
            for k in range(routing.shape[1]):
                rows = valid[:, k].nonzero().flatten()
                in_rank[rows, owner[rows, k]] = True
            tokens = torch.arange(x.shape[0], dtype=torch.int64)[:, None].expand(-1, self._world_size)
            dst_slots = torch.where(in_rank, tokens, torch.full_like(tokens, -1)).contiguous()
            capacity = int(offsets[-1])
            slot_map = torch.full((capacity if expand else 0,), -1, dtype=torch.int32)
            if expand and meta.shape[0]:
                k_ids = torch.arange(routing.shape[1])[None, :].expand_as(slots)
                row_ids = torch.arange(meta.shape[0])[:, None].expand_as(slots)
                ok = slots >= 0
                slot_map[slots[ok]] = (row_ids[ok] * routing.shape[1] + k_ids[ok]).to(torch.int32)
            layout = NativeLayout(meta, counts, offsets, prefix, int(meta.shape[0]), capacity)
            handle = NativeHandle(
                config=self._config, rank=self._rank, world_size=self._world_size, do_expand=expand, alignment=align,
                topk_idx=routing, layout=layout, dst_slots=dst_slots, send_counts=in_rank.sum(0).to(torch.int64),
                owner=self, x_dtype=x.dtype, num_sms=None, slot_map=slot_map,
            )
        layout = handle.layout
        meta = layout.recv_metadata.long()
        rows = layout.expanded_capacity if expand else layout.recv_count
        out_x = torch.zeros((rows, self._config.hidden), dtype=x.dtype) if (expand and zero_padding) else torch.empty(
            (rows, self._config.hidden), dtype=x.dtype
        )
        if expand and not zero_padding:
            out_x.fill_(float("nan"))  # make reads of uninitialised gaps visible
        out_w = None
        if weights is not None:
            out_w = torch.zeros((rows,) if expand else (rows, self._config.num_topk), dtype=torch.float32)
        for src in range(self._world_size):
            sel = (meta[:, 0] == src).nonzero().flatten()
            if sel.numel() == 0:
                continue
            tok = meta[sel, 1]
            src_x, src_w = gathered[src]["x"], gathered[src]["w"]
            if expand:
                slots = meta[sel, 2:]
                ok = slots >= 0
                rep_rows = ok.nonzero()
                out_x[slots[ok]] = src_x[tok[rep_rows[:, 0]]]
                if out_w is not None:
                    out_w[slots[ok]] = src_w[tok[rep_rows[:, 0]], rep_rows[:, 1]]
            else:
                out_x[sel] = src_x[tok]
                if out_w is not None:
                    out_w[sel] = src_w[tok]
        return NativeDispatchResult(
            x=out_x,
            topk_idx=None if expand else meta[:, 2:].contiguous(),
            topk_weights=out_w,
            handle=handle,
            event=CpuEvent() if async_op else None,
        )

    def combine(self, x, handle, *, weights=None, bias=None, previous_event=None, async_op=False, num_sms=None) -> NativeCombineResult:
        if self._closed:
            raise RuntimeError("CpuBuffer is closed")
        if handle.owner is not self:
            raise ValueError("combine handle belongs to another buffer")
        validate_combine_inputs(self._config, handle, x, weights, bias, torch.device("cpu"))
        cfg, K = self._config, self._config.num_topk
        meta = handle.layout.recv_metadata.long()
        separate = handle.do_expand and not self._allow_multiple_reduction
        # What this rank returns to every source: (token, partition k, bf16 row) triples + weight scalars.
        parcels = [dict(tok=[], part=[], rows=[], wtok=[], wk=[], wval=[]) for _ in range(self._world_size)]
        for r in range(meta.shape[0]):
            src, tok = int(meta[r, 0]), int(meta[r, 1])
            v = meta[r, 2:]
            ks = (v >= 0).nonzero().flatten().tolist()
            if not ks:
                continue
            p = parcels[src]
            if handle.do_expand:
                if separate:
                    for k in ks:
                        p["tok"].append(tok), p["part"].append(k), p["rows"].append(x[v[k]])
                else:
                    acc = torch.zeros(cfg.hidden, dtype=torch.float32)
                    for k in ks:
                        acc += x[v[k]].float()
                    p["tok"].append(tok), p["part"].append(ks[0]), p["rows"].append(acc.to(x.dtype))
                if weights is not None:
                    for k in ks:
                        p["wtok"].append(tok), p["wk"].append(k), p["wval"].append(float(weights[v[k]]))
            else:
                p["tok"].append(tok), p["part"].append(ks[0]), p["rows"].append(x[r])
                if weights is not None:
                    for k in ks:
                        p["wtok"].append(tok), p["wk"].append(k), p["wval"].append(float(weights[r, k]))
        for p in parcels:
            p["rows"] = torch.stack(p["rows"]) if p["rows"] else torch.empty((0, cfg.hidden), dtype=x.dtype)
        everything = bootstrap.gather_objects(self._group, parcels)
        T = handle.topk_idx.shape[0]
        # Sum partitions in ascending k for each token (FP32), bias once, one rounding.
        buckets = torch.zeros((K, T, cfg.hidden), dtype=torch.float32)
        out_w = torch.zeros((T, K), dtype=torch.float32) if weights is not None else None
        for dst in range(self._world_size):
            p = everything[dst][self._rank]
            if len(p["tok"]):
                buckets[torch.tensor(p["part"]), torch.tensor(p["tok"])] = p["rows"].float()
            if out_w is not None and len(p["wtok"]):
                out_w[torch.tensor(p["wtok"]), torch.tensor(p["wk"])] = torch.tensor(p["wval"], dtype=torch.float32)
        acc = torch.zeros((T, cfg.hidden), dtype=torch.float32)
        for k in range(K):
            acc += buckets[k]
        if bias is not None:
            acc += bias.float()
        return NativeCombineResult(x=acc.to(x.dtype), topk_weights=out_w, event=CpuEvent() if async_op else None)

    def barrier(self):
        dist.barrier(group=self._group)

    def close(self):
        if self._closed:
            return
        dist.barrier(group=self._group)
        self._closed = True

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
