"""NCCL baseline dispatcher: padded AllGather x3 + fp32 ReduceScatter through
``torch.distributed``.  This is the path to beat, kept with the behaviour of the reference's
``NCCLBencher`` (bench_nccl.py:31-175): ranks are padded to the per-step maximum count (found
with one all-reduce at set-up time, outside the timed region), the gathered layout is
rank-major padded, and the combine runs in fp32.  No kernel of this repository is involved.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..config import Config
from .base import Dispatcher


class NCCLDispatcher(Dispatcher):
    name = "nccl"
    num_sms = -1

    def __init__(self, cfg: Config, group, device=None):
        super().__init__(cfg, group, device)
        self.kernel_launches_per_step = lambda nl: 0   # library kernels only

    def build(self):
        cfg, dev = self.cfg, self.device
        cap, g, H, K = max(cfg.per_rank_cap, 1), max(cfg.global_cap, 1), cfg.hidden, cfg.topk
        self.cap = cap
        self.send = [torch.zeros(cap, H, dtype=torch.bfloat16, device=dev),
                     torch.zeros(cap, K, dtype=torch.int64, device=dev),
                     torch.zeros(cap, K, dtype=torch.float32, device=dev)]
        self.gathered = [torch.empty(g, H, dtype=torch.bfloat16, device=dev),
                         torch.empty(g, K, dtype=torch.int64, device=dev),
                         torch.empty(g, K, dtype=torch.float32, device=dev)]
        self.partial = torch.randn(g, H, dtype=torch.float32, device=dev)
        self.reduced = torch.empty(cap, H, dtype=torch.float32, device=dev)
        self.n = 0
        self.pad_to = 0
        self._built = True

    def setup_batch(self, hidden, topk_idx, topk_weights):
        n = hidden.shape[0]
        mx = torch.tensor([n], device=self.device, dtype=torch.int64)
        dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=self.group)      # host sync, set-up only
        self.n, self.pad_to = n, int(mx.item())
        for buf, src in zip(self.send, (hidden, topk_idx, topk_weights)):
            buf[:n] = src.to(buf.dtype)
            buf[n:self.pad_to] = 0

    @property
    def out(self):
        return self.reduced[:self.n]

    def dispatch(self):
        p, w = self.pad_to, self.cfg.ep_size
        for dst, src in zip(self.gathered, self.send):
            dist.all_gather_into_tensor(dst[:p * w], src[:p], group=self.group)

    def combine(self):
        p, w = self.pad_to, self.cfg.ep_size
        dist.reduce_scatter_tensor(self.reduced[:p], self.partial[:p * w], group=self.group)

    def functional_roundtrip(self, hidden, topk_idx):
        w, rank = self.cfg.ep_size, self.cfg.rank
        epr = self.cfg.num_experts // w
        n = hidden.shape[0]
        self.setup_batch(hidden, topk_idx, torch.zeros(n, self.cfg.topk, device=self.device))
        p = self.pad_to
        dist.all_gather_into_tensor(self.gathered[0][:p * w], self.send[0][:p], group=self.group)
        dist.all_gather_into_tensor(self.gathered[1][:p * w], self.send[1][:p], group=self.group)
        gr = self.gathered[1][:p * w]
        hit = ((gr >= rank * epr) & (gr < (rank + 1) * epr)).any(dim=1, keepdim=True)
        # padded rows carry zeros, so whatever their routing says they add nothing
        self.partial[:p * w] = torch.where(hit, self.gathered[0][:p * w].float(), torch.zeros((), device=self.device))
        dist.reduce_scatter_tensor(self.reduced[:p], self.partial[:p * w], group=self.group)
        return self.reduced[:n]

    def validate(self):
        """Round trip == m * x with random tokens at B = 2*ep and B = 1 (bench_nccl.py:121-153)."""
        w, rank, dev = self.cfg.ep_size, self.cfg.rank, self.device
        H, K, E = self.cfg.hidden, self.cfg.topk, self.cfg.num_experts
        epr = E // w
        results = []
        for B in (w * 2, 1):
            n = self._validation_counts(B)[rank]
            gen = torch.Generator(device=dev).manual_seed(990701 + B + rank * 149)
            x = torch.randn(n, H, generator=gen, device=dev).to(torch.bfloat16)
            idx = (torch.stack([torch.randperm(E, generator=gen, device=dev)[:K] for _ in range(n)])
                   if n else torch.empty(0, K, dtype=torch.int64, device=dev))
            got = self.functional_roundtrip(x, idx).float()
            torch.cuda.synchronize()
            if n:
                m = torch.tensor([torch.unique(idx[t] // epr).numel() for t in range(n)], device=dev,
                                 dtype=torch.float32).view(n, 1)
                ref = m * x.float()
                ok = bool(torch.allclose(got, ref, rtol=0.03, atol=0.05))
                detail = f"n={n} max|got-m*x|={float((got - ref).abs().max()):.4f}"
            else:
                ok, detail = True, "n=0 (idle rank still joins every collective)"
            results.append((f"NCCL dispatch->combine   B={B:<4d}", ok, detail))
        return results
