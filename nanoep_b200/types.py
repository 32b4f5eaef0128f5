"""Result and handle records returned by dispatch/combine.

Field names follow the reference's dataclasses (nano_ep/backends/cuda.py:23-62) so
code written against that API reads the same attributes here.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from .config import EPConfig


@dataclass
class NativeLayout:
    """Receive-side routing metadata of one dispatch.

    recv_metadata: int32 ``[N, K+2]``; row = ``[src_rank, src_token, v_0..v_{K-1}]`` where
        ``v_k`` is the local expert id (compact layout) or the expert-major slot (expanded
        layout) of choice k, ``-1`` when that choice is masked or lives on another rank.
    expert_counts: int64 ``[L]`` real assignments per local expert.
    expert_offsets: int64 ``[L+1]`` padded exclusive offsets; the last entry is C.
    recv_rank_prefix: int64 ``[R]`` inclusive count of receive rows by source rank.
    recv_count / expanded_capacity: host integers N and C.
    """

    recv_metadata: torch.Tensor
    expert_counts: torch.Tensor
    expert_offsets: torch.Tensor
    recv_rank_prefix: torch.Tensor
    recv_count: int
    expanded_capacity: int

    # Convenience views matching the reference's documented layout table (docs/api.md:62-70).
    @property
    def src_ranks(self) -> torch.Tensor:
        return self.recv_metadata[:, 0].long()

    @property
    def src_tokens(self) -> torch.Tensor:
        return self.recv_metadata[:, 1].long()


@dataclass
class NativeHandle:
    """Snapshot of one routing decision; pass it back for cached dispatch and for combine."""

    config: EPConfig
    rank: int
    world_size: int
    do_expand: bool
    alignment: int
    topk_idx: torch.Tensor
    layout: NativeLayout
    dst_slots: torch.Tensor
    send_counts: torch.Tensor
    owner: Any
    x_dtype: torch.dtype
    num_sms: int | None = None
    # expanded layout: int32 [C], slot -> receive_row * K + k, -1 for padding; empty for compact
    slot_map: torch.Tensor | None = None
    # native-side copy of the metadata (CUDA backend): lets cached dispatch and combine pass one object
    native_state: Any = None

    @property
    def local_topk_idx(self) -> torch.Tensor:
        """int64 ``[N, K]`` local expert ids (``-1`` elsewhere), for either layout."""
        meta = self.layout.recv_metadata[:, 2:].long()
        if not self.do_expand:
            return meta
        offsets = self.layout.expert_offsets
        expert = torch.bucketize(meta.clamp(min=0), offsets[1:].to(meta.device), right=True)
        return torch.where(meta >= 0, expert, torch.full_like(meta, -1))

    @property
    def expanded_slots(self) -> torch.Tensor:
        """int64 ``[N, K]`` expert-major slots (expanded) or an empty tensor (compact)."""
        if not self.do_expand:
            return self.layout.recv_metadata.new_empty((0,), dtype=torch.int64)
        return self.layout.recv_metadata[:, 2:].long()


@dataclass
class NativeDispatchResult:
    x: torch.Tensor
    topk_idx: torch.Tensor | None
    topk_weights: torch.Tensor | None
    handle: NativeHandle
    event: Any | None


@dataclass
class NativeCombineResult:
    x: torch.Tensor
    topk_weights: torch.Tensor | None
    event: Any | None
