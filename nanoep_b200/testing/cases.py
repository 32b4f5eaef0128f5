"""Small reproducible routing cases for tests.

The same case kinds as the reference generator (nano_ep/testing/cases.py:18-56): random,
empty (last rank sends nothing), masked (every choice -1), skew (everyone picks the same
experts) and mixed; plus the routing generators used by the benchmark configurations
(balanced softmax top-k, Zipf-skewed with masked slots).  Gate weights are deliberately
non-zero at masked slots so a backend that forwards them blindly is caught.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

KINDS = ("random", "empty", "masked", "skew", "mixed")


@dataclass
class Case:
    xs: list[torch.Tensor]
    indices: list[torch.Tensor]
    weights: list[torch.Tensor]
    num_experts: int
    num_topk: int
    hidden: int
    capacity: int

    @property
    def world_size(self) -> int:
        return len(self.xs)


def make_case(
    world_size: int = 2,
    *,
    seed: int = 0,
    kind: str = "random",
    dtype: torch.dtype = torch.bfloat16,
    hidden: int = 256,
    experts_per_rank: int = 3,
    topk: int = 3,
    tokens: int = 5,
) -> Case:
    if kind not in KINDS:
        raise ValueError(f"unknown case kind {kind!r}")
    gen = torch.Generator().manual_seed(seed)
    experts = world_size * experts_per_rank
    topk = min(topk, experts)
    xs, indices, weights = [], [], []
    for rank in range(world_size):
        count = max(0, tokens - rank % 4)
        if kind == "empty" and rank == world_size - 1:
            count = 0
        x = torch.randn(count, hidden, generator=gen, dtype=torch.float32).to(dtype)
        idx = torch.empty((count, topk), dtype=torch.int64)
        for t in range(count):
            if kind == "skew":
                chosen = torch.arange(topk - 1, -1, -1, dtype=torch.int64)
            elif kind == "mixed" and t % 2 == 0:
                base = (t % world_size) * experts_per_rank
                chosen = (base + torch.arange(topk, dtype=torch.int64).roll(1)) % experts
            else:
                chosen = torch.randperm(experts, generator=gen)[:topk]
            chosen = chosen.clone()
            if kind == "masked":
                chosen[:] = -1
            elif kind in ("random", "mixed") and t == 0 and topk > 1:
                chosen[1] = -1
            idx[t] = chosen
        w = torch.randn(count, topk, generator=gen, dtype=torch.float32) + 0.3
        xs.append(x)
        indices.append(idx)
        weights.append(w)
    return Case(xs, indices, weights, experts, topk, hidden, max(1, tokens))


def balanced_routing(tokens: int, num_experts: int, topk: int, *, seed: int, device="cpu"):
    """Top-k of softmax(N(0,1) logits); weights renormalised to sum to one (fp32)."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    logits = torch.randn(tokens, num_experts, generator=gen, dtype=torch.float32)
    probs = torch.softmax(logits, dim=-1)
    w, idx = probs.topk(topk, dim=-1)
    w = w / w.sum(-1, keepdim=True)
    return idx.to(torch.int64).to(device), w.to(device)


def zipf_routing(tokens: int, num_experts: int, topk: int, *, seed: int, s: float = 1.2, mask_fraction: float = 0.1, device="cpu"):
    """Distinct experts drawn with Zipf(s) popularity under a seeded permutation; a fraction masked to -1."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    ranks = torch.arange(1, num_experts + 1, dtype=torch.float64)
    popularity = (1.0 / ranks.pow(s))[torch.randperm(num_experts, generator=gen)]
    probs = (popularity / popularity.sum()).expand(tokens, -1)
    idx = torch.multinomial(probs, topk, replacement=False, generator=gen).to(torch.int64)
    w = torch.rand(tokens, topk, generator=gen, dtype=torch.float32) + 0.1
    w = w / w.sum(-1, keepdim=True)
    if mask_fraction > 0:
        drop = torch.rand(tokens, topk, generator=gen) < mask_fraction
        idx = idx.masked_fill(drop, -1)
    return idx.to(device), w.to(device)


def uniform_routing(tokens: int, num_experts: int, topk: int, *, seed: int, device="cpu"):
    """Uniformly random distinct experts per token, uniform weights."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    scores = torch.rand(tokens, num_experts, generator=gen)
    idx = scores.topk(topk, dim=-1).indices.to(torch.int64)
    w = torch.full((tokens, topk), 1.0 / topk, dtype=torch.float32)
    return idx.to(device), w.to(device)
