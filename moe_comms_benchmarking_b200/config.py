"""Run configuration.

Same fields and derived properties as the reference's ``Config`` (common.py:28-47), with
the model shape made configurable (the reference hard-codes 512/22/1024, common.py:22-24)
so that the DeepSeek-V3 shape and the CPU plumbing shape are expressible.
"""
from __future__ import annotations

from dataclasses import dataclass

NUM_EXPERTS = 512
TOPK = 22
HIDDEN = 1024


@dataclass
class Config:
    num_experts: int = NUM_EXPERTS
    topk: int = TOPK
    hidden: int = HIDDEN
    intermediate: int = 1024          # SwiGLU expert width (only used with real experts)
    ep_size: int = 1
    rank: int = 0
    local_rank: int = 0
    per_rank_cap: int = 0             # most tokens a single rank can hold: ceil(max_B / ep)
    seed: int = 1234
    routing: str = "uniform"          # uniform | zipf
    probs: str = "softmax"            # softmax | sigmoid
    counts: str = "balanced"          # balanced | multinomial (one rank forced to 0 tokens)

    def __post_init__(self):
        if self.ep_size < 1:
            raise ValueError("ep_size must be >= 1")
        if self.num_experts % self.ep_size != 0:
            raise ValueError(f"num_experts={self.num_experts} is not divisible by ep_size={self.ep_size}")
        if self.topk > self.num_experts:
            raise ValueError("topk exceeds num_experts")

    @property
    def num_local_experts(self) -> int:
        return self.num_experts // self.ep_size

    @property
    def global_cap(self) -> int:
        return self.per_rank_cap * self.ep_size
