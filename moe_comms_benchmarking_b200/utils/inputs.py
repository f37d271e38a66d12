"""Seeded synthetic inputs for the decode benchmark.

``make_inputs`` reproduces the contract of the reference generator (common.py:85-112):
deterministic in (seed, global batch, rank); ``topk`` DISTINCT experts per token; fp32
weights; bf16 hidden states; empty tensors on a rank that holds no tokens.  On top of the
reference's uniform routing it offers Zipf-skewed expert popularity, sigmoid-normalised
weights (DeepSeek-V3 style) and multinomial per-rank token counts with one idle rank.
"""
from __future__ import annotations

import torch

from ..config import Config
from ..parallel.dist import all_rank_counts


def rank_counts(cfg: Config, global_b: int) -> list[int]:
    """Tokens per rank for a global batch.  ``balanced`` is the reference's split
    (common.py:71-81).  ``multinomial`` draws the split from a seeded multinomial over all
    ranks but one (the last rank of a seeded permutation gets no tokens), clipped to the
    per-rank capacity; identical on every rank."""
    w = cfg.ep_size
    if cfg.counts == "balanced" or w == 1:
        return all_rank_counts(global_b, w)
    if cfg.counts != "multinomial":
        raise ValueError(f"unknown counts mode {cfg.counts!r}")
    gen = torch.Generator().manual_seed(cfg.seed * 7919 + global_b)
    perm = torch.randperm(w, generator=gen)
    active = perm[:-1]
    draws = torch.multinomial(torch.ones(w - 1), global_b, replacement=True, generator=gen)
    counts = torch.zeros(w, dtype=torch.int64)
    counts.index_add_(0, active[draws], torch.ones(global_b, dtype=torch.int64))
    cap = cfg.per_rank_cap if cfg.per_rank_cap > 0 else global_b
    # Move overflow beyond the capacity to the emptiest active ranks (keeps sum == B when it fits).
    over = int((counts - cap).clamp(min=0).sum())
    counts.clamp_(max=cap)
    while over > 0:
        room = [(int(counts[r]), int(r)) for r in active.tolist() if counts[r] < cap]
        if not room:
            break
        _, r = min(room)
        counts[r] += 1
        over -= 1
    return [int(c) for c in counts]


def expert_log_popularity(cfg: Config, device) -> torch.Tensor | None:
    """log p_e for Zipf(s=1.2) popularity over a seeded permutation of the experts."""
    if cfg.routing == "uniform":
        return None
    if cfg.routing != "zipf":
        raise ValueError(f"unknown routing mode {cfg.routing!r}")
    gen = torch.Generator().manual_seed(cfg.seed * 104729 + 17)
    perm = torch.randperm(cfg.num_experts, generator=gen)
    ranks = torch.empty(cfg.num_experts, dtype=torch.float64)
    ranks[perm] = torch.arange(1, cfg.num_experts + 1, dtype=torch.float64)
    logp = -1.2 * torch.log(ranks)
    return (logp - torch.logsumexp(logp, 0)).to(torch.float32).to(device)


def make_inputs(cfg: Config, global_b: int, device, n: int | None = None):
    """This rank's ``(hidden[n,H] bf16, topk_idx[n,K] int64, topk_weights[n,K] fp32)``."""
    if n is None:
        n = rank_counts(cfg, global_b)[cfg.rank]
    K, E, H = cfg.topk, cfg.num_experts, cfg.hidden
    device = torch.device(device)
    gen = torch.Generator(device=device).manual_seed(cfg.seed + global_b * 131 + cfg.rank)
    hidden = torch.randn((n, H), device=device, dtype=torch.float32, generator=gen).to(torch.bfloat16)
    if n == 0:
        return (hidden, torch.empty((0, K), device=device, dtype=torch.int64),
                torch.empty((0, K), device=device, dtype=torch.float32))
    u = torch.rand((n, E), device=device, generator=gen)
    logp = expert_log_popularity(cfg, device)
    if logp is None:
        sel, topk_idx = torch.topk(u, K, dim=-1)            # K distinct uniform experts
    else:
        # Gumbel top-k: K distinct experts drawn without replacement with probability ~ p_e.
        g = -torch.log(-torch.log(u.clamp(1e-9, 1 - 1e-7)))
        _, topk_idx = torch.topk(logp.unsqueeze(0) + g, K, dim=-1)
        sel = torch.gather(u, 1, topk_idx)
    if cfg.probs == "softmax":
        w = torch.softmax(sel, dim=-1)
    elif cfg.probs == "sigmoid":
        s = torch.sigmoid(torch.randn((n, K), device=device, generator=gen))
        w = s / s.sum(dim=-1, keepdim=True)
    else:
        raise ValueError(f"unknown probs mode {cfg.probs!r}")
    return hidden, topk_idx.to(torch.int64), w.to(torch.float32)


def size_mb(shape, dtype) -> int:
    """Bytes of a tensor rounded up to whole MiB, at least 1 (common.py:116-118)."""
    n = 1
    for s in shape:
        n *= int(s)
    nbytes = n * torch.empty((), dtype=dtype).element_size()
    return max(1, (nbytes + (1 << 20) - 1) >> 20)
