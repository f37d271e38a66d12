"""NCCL baseline dispatcher: padded AllGather x3 + fp32 ReduceScatter through
``torch.distributed``.  This is the path to beat, kept with the behaviour of the reference's
``NCCLBencher`` (bench_nccl.py:31-175): ranks are padded to the per-step maximum count (found
with one all-reduce at set-up time, outside the timed region), the gathered layout is
rank-major padded, and the combine runs in fp32.  No kernel of this repository is involved.

``NCCLSwiGLUDispatcher`` is an EXTENDED baseline that the reference does not have (its expert is
the identity, bench_nccl.py:106-109): the same NCCL transport around real SwiGLU experts computed
with library GEMMs (``torch._grouped_mm`` when this PyTorch has it for the device, else one
``torch.mm`` pair per expert).  It exists only to give the fused expert path of this repository
something to be compared with; it is never used by a product path.
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


class NCCLSwiGLUDispatcher(NCCLDispatcher):
    """NCCL all-gather x3 -> library grouped GEMMs (SwiGLU FFN of this rank's experts) -> fp32 NCCL
    reduce-scatter.  Extended baseline, labelled as such wherever it is reported.

    Per layer, with static shapes so that the step can be captured as a CUDA graph: the (token, k)
    entries of the gathered routing are sorted by local expert (entries of other ranks' experts sort
    last), the first ``num_pairs`` entries are this rank's work (``num_pairs`` and the per-expert
    counts are read on the host once per batch in ``setup_batch``, outside the timed region, like the
    pad count of the plain NCCL baseline), the token rows are gathered, multiplied expert by expert,
    weighted and summed into the fp32 buffer that the reduce-scatter consumes."""
    name = "nccl-swiglu"

    def __init__(self, cfg: Config, group, num_layers: int = 88, weight_budget_gb: float = 48.0, weight_seed: int = 7,
                 device=None):
        super().__init__(cfg, group, device)
        self.num_layers, self.weight_budget_gb, self.weight_seed = num_layers, weight_budget_gb, weight_seed

    def build(self):
        super().build()
        cfg, dev = self.cfg, self.device
        E, H, I = cfg.num_local_experts, cfg.hidden, cfg.intermediate
        per_layer = E * 3 * H * I * 2
        sets = max(1, min(self.num_layers, int(self.weight_budget_gb * 2**30 // per_layer)))
        self.w_gate_up, self.w_down = [], []
        for s in range(sets):       # the same values as ExpertWeights of the fused dispatcher with this seed
            g = torch.Generator(device=dev).manual_seed(self.weight_seed * 100003 + s * 1009 + cfg.rank)
            self.w_gate_up.append((torch.randn(E, 2 * I, H, device=dev, generator=g) * 0.02).to(torch.bfloat16))
            self.w_down.append((torch.randn(E, H, I, device=dev, generator=g) * 0.02).to(torch.bfloat16))
        self.grouped = False
        if hasattr(torch, "_grouped_mm"):
            try:        # does this PyTorch have the grouped kernel for this device?
                a = torch.zeros(32, H, dtype=torch.bfloat16, device=dev)
                offs = torch.tensor([16, 32], dtype=torch.int32, device=dev)
                torch._grouped_mm(a, self.w_gate_up[0][:2].transpose(1, 2), offs=offs)
                torch.cuda.synchronize()
                self.grouped = True
            except Exception:
                self.grouped = False
        self.layer_index = 0

    def setup_batch(self, hidden, topk_idx, topk_weights):
        super().setup_batch(hidden, topk_idx, topk_weights)
        # one untimed dispatch to learn the static shapes of this batch
        self.dispatch()
        keys = self._keys()
        E = self.cfg.num_local_experts
        counts = torch.bincount(keys, minlength=E + 1)[:E]
        self.counts_host = counts.tolist()                      # host sync, set-up only
        self.num_pairs = int(sum(self.counts_host))
        self.offs = torch.cumsum(counts, 0).to(torch.int32)

    def _keys(self):
        """Local expert of every gathered (token, k) entry; entries of other ranks (and of padded rows) get E_loc."""
        cfg, p, w = self.cfg, self.pad_to, self.cfg.ep_size
        E = cfg.num_local_experts
        idx = self.gathered[1][:p * w] - cfg.rank * E
        valid = (self.gathered[2][:p * w] != 0) | (self.gathered[0][:p * w].abs().sum(1, keepdim=True) != 0)
        local = (idx >= 0) & (idx < E) & valid
        return torch.where(local, idx, torch.full_like(idx, E)).flatten()

    def experts(self, layer: int = 0):
        cfg, p, w = self.cfg, self.pad_to, self.cfg.ep_size
        K, P = cfg.topk, self.num_pairs
        s = layer % len(self.w_gate_up)
        self.partial[:p * w].zero_()
        if P == 0:
            return
        order = torch.argsort(self._keys(), stable=True)[:P]
        tok = order // K
        xs = self.gathered[0][:p * w][tok]
        prob = self.gathered[2][:p * w].flatten()[order].unsqueeze(1)
        I = cfg.intermediate
        if self.grouped:
            gu = torch._grouped_mm(xs, self.w_gate_up[s].transpose(1, 2), offs=self.offs)
            act = (torch.nn.functional.silu(gu[:, :I].float()) * gu[:, I:].float()).to(torch.bfloat16)
            y = torch._grouped_mm(act, self.w_down[s].transpose(1, 2), offs=self.offs)
        else:
            y = torch.empty(P, cfg.hidden, dtype=torch.bfloat16, device=self.device)
            r0 = 0
            for e, c in enumerate(self.counts_host):
                if c:
                    gu = xs[r0:r0 + c] @ self.w_gate_up[s][e].t()
                    act = (torch.nn.functional.silu(gu[:, :I].float()) * gu[:, I:].float()).to(torch.bfloat16)
                    y[r0:r0 + c] = act @ self.w_down[s][e].t()
                    r0 += c
        self.partial[:p * w].index_add_(0, tok, y.float() * prob)

    def step(self):
        self.dispatch()
        self.experts(self.layer_index)
        self.combine()

    def decode_step(self, num_layers: int):
        for l in range(num_layers):
            self.layer_index = l
            self.step()
        self.layer_index = 0

    def functional_roundtrip(self, hidden, topk_idx):
        raise NotImplementedError("the extended baseline computes real experts; compare it with the fused dispatcher")

    def validate(self):
        """One layer against the CPU oracle (weights of all ranks regenerated from their seeds)."""
        from ..ops import oracle
        from ..utils.inputs import make_inputs
        cfg, rank, dev = self.cfg, self.cfg.rank, self.device
        E, H, I = cfg.num_local_experts, cfg.hidden, cfg.intermediate
        results = []
        for B in (cfg.ep_size * 2, 1):
            n = self._validation_counts(B)[rank]
            h, i, w = make_inputs(cfg, B, dev, n=n)
            self.setup_batch(h, i, w)
            self.step()
            torch.cuda.synchronize()
            if n:
                wgu, wd = [], []
                for r in range(cfg.ep_size):
                    g = torch.Generator(device=dev).manual_seed(self.weight_seed * 100003 + r)
                    wgu.append((torch.randn(E, 2 * I, H, device=dev, generator=g) * 0.02).to(torch.bfloat16).cpu())
                    wd.append((torch.randn(E, H, I, device=dev, generator=g) * 0.02).to(torch.bfloat16).cpu())
                ref = oracle.moe_layer(h.cpu(), i.cpu(), w.cpu(), torch.cat(wgu), torch.cat(wd))
                got = self.out.float().cpu()
                scale = float(ref.abs().max()) + 1e-6
                err = float((got - ref).abs().max())
                ok, detail = err / scale < 0.05, f"n={n} max|got-ref|={err:.5f} ({100 * err / scale:.2f}% of {scale:.4f}); grouped_mm={self.grouped}"
            else:
                ok, detail = True, "n=0 (idle rank still runs its experts on other ranks' tokens)"
            results.append((f"NCCL + library SwiGLU vs oracle B={B:<4d}", bool(ok), detail))
        return results
