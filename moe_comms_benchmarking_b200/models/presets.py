"""Model shape presets.  The reference knows one shape only (common.py:22-24, Nemotron-Super:
512 experts, top-22, hidden 1024, 88 MoE layers, run.py:52-53)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class MoEShape:
    name: str
    num_experts: int
    topk: int
    hidden: int
    intermediate: int
    num_layers: int
    probs: str = "softmax"


PRESETS = {
    "nemotron-super": MoEShape("nemotron-super", 512, 22, 1024, 1024, 88, "softmax"),
    "deepseek-v3": MoEShape("deepseek-v3", 256, 8, 7168, 2048, 58, "sigmoid"),
    "tiny-cpu": MoEShape("tiny-cpu", 16, 4, 128, 128, 2, "softmax"),
}


def get_preset(name: str) -> MoEShape:
    try:
        return PRESETS[name]
    except KeyError:
        raise ValueError(f"unknown model preset {name!r}; choose from {sorted(PRESETS)}") from None
