"""CPU dispatcher over gloo: the dense algorithm (padded AllGather -> identity expert ->
ReduceScatter emulated as all_reduce + slice) with no GPU.  It exists so the host-side
logic (token split, padding, masks, validation verdicts, CSV) is exercised as real
multi-process ranks on a machine without GPUs; the reference has no such path
(its only check needs NVLink GPUs, README.md:68-78).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..config import Config
from .base import Dispatcher


class GlooDenseDispatcher(Dispatcher):
    name = "gloo"
    num_sms = -1

    def __init__(self, cfg: Config, group, dtype=torch.float32):
        super().__init__(cfg, group, torch.device("cpu"))
        self.dtype = dtype

    def build(self):
        cfg = self.cfg
        cap, g, H, K = max(cfg.per_rank_cap, 1), max(cfg.global_cap, 1), cfg.hidden, cfg.topk
        self.cap = cap
        self.pad_h = torch.zeros(cap, H, dtype=self.dtype)
        self.pad_r = torch.zeros(cap, K, dtype=torch.int64)
        self.pad_p = torch.zeros(cap, K, dtype=torch.float32)
        self.g_h = torch.zeros(g, H, dtype=self.dtype)
        self.g_r = torch.zeros(g, K, dtype=torch.int64)
        self.g_p = torch.zeros(g, K, dtype=torch.float32)
        self.partial = torch.zeros(g, H, dtype=torch.float32)
        self.n = self.pad_to = 0
        self._built = True

    def setup_batch(self, hidden, topk_idx, topk_weights):
        n = hidden.shape[0]
        mx = torch.tensor([n], dtype=torch.int64)
        dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=self.group)
        self.n, self.pad_to = n, int(mx.item())
        p = self.pad_to
        self.pad_h[:p] = 0
        self.pad_r[:p] = 0
        self.pad_p[:p] = 0
        self.pad_h[:n] = hidden.to(self.dtype)
        self.pad_r[:n] = topk_idx
        self.pad_p[:n] = topk_weights

    def dispatch(self):
        p, w = self.pad_to, self.cfg.ep_size
        if p == 0:
            return
        for dst, src in ((self.g_h, self.pad_h), (self.g_r, self.pad_r), (self.g_p, self.pad_p)):
            dist.all_gather_into_tensor(dst[:p * w], src[:p].contiguous(), group=self.group)

    def expert(self):
        """Masked identity expert: keep a gathered token iff it routed to a local expert."""
        p, w, rank = self.pad_to, self.cfg.ep_size, self.cfg.rank
        epr = self.cfg.num_experts // w
        gr = self.g_r[:p * w]
        hit = ((gr >= rank * epr) & (gr < (rank + 1) * epr)).any(dim=1, keepdim=True)
        self.partial[:p * w] = torch.where(hit, self.g_h[:p * w].float(), torch.zeros(()))

    def combine(self):
        p, w, rank = self.pad_to, self.cfg.ep_size, self.cfg.rank
        if p == 0:
            self.out = torch.zeros(0, self.cfg.hidden)
            return
        total = self.partial[:p * w].clone()
        dist.all_reduce(total, op=dist.ReduceOp.SUM, group=self.group)     # reduce-scatter = all_reduce + slice
        self.out = total[rank * p: rank * p + self.n]

    def step(self):
        self.dispatch()
        self.expert()
        self.combine()

    def functional_roundtrip(self, hidden, topk_idx):
        n = hidden.shape[0]
        self.setup_batch(hidden, topk_idx, torch.ones(n, self.cfg.topk))
        self.step()
        return self.out

    def validate(self):
        from ..ops import oracle
        w, rank = self.cfg.ep_size, self.cfg.rank
        H, K, E = self.cfg.hidden, self.cfg.topk, self.cfg.num_experts
        results = []
        for B in (w * 2, 1):
            n = self._validation_counts(B)[rank]
            gen = torch.Generator().manual_seed(440701 + B + rank * 149)
            x = torch.randn(n, H, generator=gen)
            idx = (torch.stack([torch.randperm(E, generator=gen)[:K] for _ in range(n)])
                   if n else torch.empty(0, K, dtype=torch.int64))
            got = self.functional_roundtrip(x, idx)
            if n:
                ref = oracle.roundtrip_identity(x, idx, E, w)
                ok = bool(torch.allclose(got, ref, rtol=1e-5, atol=1e-5))
                detail = f"n={n} max|got-m*x|={float((got - ref).abs().max()):.2e}"
            else:
                ok, detail = True, "n=0 (idle rank still joins every collective)"
            results.append((f"gloo dispatch->combine   B={B:<4d}", ok, detail))
        return results
