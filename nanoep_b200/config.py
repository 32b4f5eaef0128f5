"""Static description of one expert-parallel group.

Same four fields and the same validation rules as the reference's ``EPConfig``
(nano_ep/config.py:4-35): all dimensions positive and ``num_topk`` no larger than
``min(32, num_experts)``.
"""

from dataclasses import dataclass

MAX_TOPK = 32


@dataclass(frozen=True)
class EPConfig:
    """Geometry shared by every rank of an expert-parallel group.

    num_experts: global expert count E; rank r owns the contiguous block
        ``[r * E / R, (r + 1) * E / R)``.
    num_topk: routing choices per token (K).
    hidden: row width H in elements (bf16); the CUDA backend wants H % 256 == 0.
    num_max_tokens_per_rank: upper bound Tmax on the tokens a rank may submit in
        one dispatch; it sizes the peer window.
    """

    num_experts: int
    num_topk: int
    hidden: int
    num_max_tokens_per_rank: int

    def __post_init__(self):
        dims = (self.num_experts, self.num_topk, self.hidden, self.num_max_tokens_per_rank)
        if any(isinstance(v, bool) or not isinstance(v, int) for v in dims):
            raise TypeError("EPConfig fields must be integers")
        if min(dims) <= 0:
            raise ValueError("EP dimensions and token capacity must be positive")
        if self.num_topk > min(MAX_TOPK, self.num_experts):
            raise ValueError("num_topk must be <= min(32, num_experts)")

    def local_experts(self, world_size: int) -> int:
        if world_size <= 0 or self.num_experts % world_size:
            raise ValueError("num_experts must be divisible by world_size")
        return self.num_experts // world_size
