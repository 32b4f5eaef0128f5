"""CPU specification of dispatch, combine and a dense MoE.

Written from the documented semantics only; it never imports the production routing
code, the window layout or a backend, so an agreement between the two is evidence.
Plays the role of the reference's scalar-loop oracle (nano_ep/testing/oracle.py:45-210)
and keeps its result names so checks port over.

All functions take per-rank lists (``xs[r]``, ``indices[r]``, ...) describing the whole
group at once.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import torch


@dataclass
class ExpectedPlan:
    topk_idx: torch.Tensor
    token_in_rank: torch.Tensor  # bool [T, R]
    send_counts: torch.Tensor  # int64 [R]
    expert_counts: torch.Tensor  # int64 [E] (global experts, this source only)


@dataclass
class ExpectedLayout:
    src_ranks: torch.Tensor
    src_tokens: torch.Tensor
    local_topk_idx: torch.Tensor
    expert_counts: torch.Tensor
    expert_offsets: torch.Tensor
    expanded_slots: torch.Tensor
    recv_count: int
    expanded_capacity: int


@dataclass
class ExpectedBatch:
    x: torch.Tensor
    topk_idx: torch.Tensor | None
    topk_weights: torch.Tensor | None
    layout: ExpectedLayout
    rank: int
    do_expand: bool


def _owner(expert: int, local_experts: int) -> int:
    return expert // local_experts


def reference_plan(indices: torch.Tensor, num_experts: int, world_size: int) -> ExpectedPlan:
    """What one source rank sends: destination mask per token and counts."""
    local = num_experts // world_size
    tokens = indices.shape[0]
    in_rank = torch.zeros((tokens, world_size), dtype=torch.bool)
    per_expert = torch.zeros(num_experts, dtype=torch.int64)
    for t in range(tokens):
        for e in indices[t].tolist():
            if e < 0:
                continue
            per_expert[e] += 1
            in_rank[t, _owner(e, local)] = True
    return ExpectedPlan(indices.clone(), in_rank, in_rank.sum(0).to(torch.int64), per_expert)


def reference_layout(indices: Sequence[torch.Tensor], rank: int, num_experts: int, alignment: int = 1) -> ExpectedLayout:
    """Receive layout of ``rank``: rows ordered by (source rank, source token)."""
    world = len(indices)
    local = num_experts // world
    topk = indices[0].shape[1]
    lo = rank * local
    src_ranks: list[int] = []
    src_tokens: list[int] = []
    local_rows: list[list[int]] = []
    counts = [0] * local
    for src in range(world):
        for tok, row in enumerate(indices[src].tolist()):
            mine = [e - lo if lo <= e < lo + local else -1 for e in row]
            if max(mine, default=-1) < 0:
                continue
            src_ranks.append(src)
            src_tokens.append(tok)
            local_rows.append(mine)
            for e in mine:
                if e >= 0:
                    counts[e] += 1
    offsets = [0]
    for c in counts:
        offsets.append(offsets[-1] + -(-c // alignment) * alignment)
    cursor = offsets[:-1].copy()
    slots = []
    for mine in local_rows:
        out = []
        for e in mine:
            if e >= 0:
                out.append(cursor[e])
                cursor[e] += 1
            else:
                out.append(-1)
        slots.append(out)
    as_i64 = lambda v, shape=None: torch.tensor(v, dtype=torch.int64).reshape(shape) if shape else torch.tensor(v, dtype=torch.int64)
    return ExpectedLayout(
        as_i64(src_ranks),
        as_i64(src_tokens),
        as_i64(local_rows, (-1, topk)),
        as_i64(counts),
        as_i64(offsets),
        as_i64(slots, (-1, topk)),
        len(local_rows),
        offsets[-1],
    )


def reference_dispatch(
    xs: Sequence[torch.Tensor],
    indices: Sequence[torch.Tensor],
    num_experts: int,
    weights: Sequence[torch.Tensor] | None = None,
    *,
    do_expand: bool = False,
    alignment: int = 1,
) -> list[ExpectedBatch]:
    """Expected receive tensors of every rank; padding rows are zero."""
    topk = indices[0].shape[1]
    out = []
    for rank in range(len(xs)):
        lay = reference_layout(indices, rank, num_experts, alignment)
        rows = lay.expanded_capacity if do_expand else lay.recv_count
        data = xs[0].new_zeros((rows, xs[0].shape[1]))
        w_out = None
        if weights is not None:
            w_out = weights[0].new_zeros((rows,) if do_expand else (rows, topk))
        for r, (src, tok) in enumerate(zip(lay.src_ranks.tolist(), lay.src_tokens.tolist())):
            if do_expand:
                for k, slot in enumerate(lay.expanded_slots[r].tolist()):
                    if slot < 0:
                        continue
                    data[slot] = xs[src][tok]
                    if w_out is not None:
                        w_out[slot] = weights[src][tok, k]
            else:
                data[r] = xs[src][tok]
                if w_out is not None:
                    w_out[r] = weights[src][tok]
        out.append(ExpectedBatch(data, None if do_expand else lay.local_topk_idx.clone(), w_out, lay, rank, do_expand))
    return out


def reference_combine(
    outputs: Sequence[torch.Tensor],
    batches: Sequence[ExpectedBatch],
    indices: Sequence[torch.Tensor],
    weights: Sequence[torch.Tensor] | None = None,
    biases: Sequence[torch.Tensor | None] | None = None,
) -> tuple[list[torch.Tensor], list[torch.Tensor] | None]:
    """Sum every returned row at its source in FP32, add bias once, round once."""
    dtype = outputs[0].dtype
    acc_dtype = torch.float64 if dtype == torch.float64 else torch.float32
    hidden = outputs[0].shape[1]
    acc = [torch.zeros((len(idx), hidden), dtype=acc_dtype) for idx in indices]
    w_back = None if weights is None else [weights[0].new_zeros(idx.shape) for idx in indices]
    for dst, batch in enumerate(batches):
        lay = batch.layout
        for r, (src, tok) in enumerate(zip(lay.src_ranks.tolist(), lay.src_tokens.tolist())):
            if batch.do_expand:
                for k, slot in enumerate(lay.expanded_slots[r].tolist()):
                    if slot < 0:
                        continue
                    acc[src][tok] += outputs[dst][slot].to(acc_dtype)
                    if w_back is not None:
                        w_back[src][tok, k] = weights[dst][slot]
            else:
                acc[src][tok] += outputs[dst][r].to(acc_dtype)
                if w_back is not None:
                    for k, e in enumerate(lay.local_topk_idx[r].tolist()):
                        if e >= 0:
                            w_back[src][tok, k] = weights[dst][r, k]
    if biases is not None:
        for rank, bias in enumerate(biases):
            if bias is not None:
                acc[rank] += bias.to(acc_dtype)
    return [a.to(dtype) for a in acc], w_back


def dense_moe(
    xs: Sequence[torch.Tensor],
    indices: Sequence[torch.Tensor],
    weights: Sequence[torch.Tensor],
    expert_fn,
) -> list[torch.Tensor]:
    """Source-local dense answer: ``sum_k w[t,k] * expert_fn(x[t], e_k)`` in FP32.

    ``expert_fn(x_rows_fp32, expert_id)`` maps ``[n, H] -> [n, H]``.
    """
    outs = []
    for x, idx, w in zip(xs, indices, weights):
        acc = torch.zeros(x.shape, dtype=torch.float32)
        for k in range(idx.shape[1]):
            for e in idx[:, k].unique().tolist():
                if e < 0:
                    continue
                rows = (idx[:, k] == e).nonzero().flatten()
                acc[rows] += expert_fn(x[rows].float(), e) * w[rows, k, None].float()
        outs.append(acc)
    return outs
