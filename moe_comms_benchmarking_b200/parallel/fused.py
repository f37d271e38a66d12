"""Dense dispatcher with REAL experts: AllGather-V dispatch -> routing -> grouped SwiGLU FFN on
tcgen05 -> prob-weighted combine (local pre-sum + cross-rank reduce-scatter in one kernel).

The reference stops at the identity expert (bench_nvls.py:109-112 and README.md:20-23:
"dispatch -> (identity expert) -> combine"); this dispatcher is the same transport with the
expert computation the transport exists for.  Per layer and rank:

    dispatch   all-gather-V of (hidden, routing, probs)           csrc/dense.cu   agv_kernel
    route      pair lists + row tiles for this rank's experts     csrc/route.cu   route_kernel
    FC1        act = silu(x Wg^T) * (x Wu^T), token gather fused  csrc/gemm.cu    grouped_gemm_kernel<FC1>
    FC2        y = prob * (act Wd^T)                              csrc/gemm.cu    grouped_gemm_kernel<FC2>
    combine    out[t] = sum_ranks sum_local-pairs y               csrc/route.cu   combine_kernel

By default the whole layer is ONE cooperative kernel (``moe_layer_kernel`` in csrc/ffn.cu: dispatch,
grid barrier, routing, grid barrier, the grouped FFN with the weights as the M = 128 operand and both
projections in one persistent weight stream, grid barrier, combine), and a decode step is issued by
one native call (count exchange + one launch per layer).  ``layer_kernel=False`` selects the older
form with the tokens as the M operand: two kernels per layer (``dispatch_route_fc1_kernel`` and
``fc2_combine_kernel`` in csrc/gemm.cu), or five with ``fuse_dispatch=False`` / ``fuse_combine=False``.

Weights: 512 experts x 3 x 1024^2 bf16 is 3.2 GB per layer; every layer gets its own set while
they fit in ``weight_budget_gb`` per GPU, after which sets are reused round-robin (each set is
far larger than L2, so a layer still streams its weights from HBM).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..config import Config
from ..ops import _ext, oracle
from ..ops.dense import AllGatherVPlan, MetadataPlan, DEFAULT_GRID, DEFAULT_THREADS, agv_ll_stage_bytes
from ..ops.experts import (DispatchRouteFc1Plan, ExpertCombinePlan, ExpertFfnPlan, ExpertWeights, Fc2CombinePlan,
                           GroupedGemmPlan, MoeLayerPlan, RouteBuffers, RoutePlan, NUM_SMS)
from .base import Dispatcher
from .dense import resolve_ll_rows
from .symm_heap import SymmetricHeap, required_bytes


class FusedExpertDispatcher(Dispatcher):
    name = "fused"

    def __init__(self, cfg: Config, group, heap: SymmetricHeap | None = None, num_sms: int = DEFAULT_GRID,
                 threads: int = DEFAULT_THREADS, pdl: bool = True, transport: str = "auto", ll_rows: int = -1,
                 num_layers: int = 88, weight_budget_gb: float = 64.0, weight_seed: int = 7,
                 fuse_combine: bool = True, fuse_dispatch: bool = True, coop_pdl: bool = False,
                 layer_kernel: bool = True, phase_trace: bool = False, device=None):
        super().__init__(cfg, group, device)
        self.heap, self._own_heap = heap, heap is None
        self.num_sms, self.threads, self.pdl, self.transport = int(num_sms), int(threads), bool(pdl), transport
        self.ll_rows = resolve_ll_rows(cfg, ll_rows)
        self.num_layers, self.weight_budget_gb, self.weight_seed = num_layers, weight_budget_gb, weight_seed
        self.fuse_combine = bool(fuse_combine)
        self.coop_pdl = bool(coop_pdl)   # cooperative + programmatic dependent launch on the fused kernel
        self.fuse_dispatch = bool(fuse_dispatch)
        self.layer_kernel = bool(layer_kernel)
        self.phase_trace = bool(phase_trace) and self.layer_kernel
        self.kernel_launches_per_step = lambda nl: 1 + (
            1 if self.layer_kernel else 5 - int(self.fuse_combine) - 2 * int(self.fuse_dispatch)) * nl

    @staticmethod
    def heap_specs(cfg: Config, ll_rows: int = -1):
        g, H, K = max(cfg.global_cap, 1), cfg.hidden, cfg.topk
        ll = resolve_ll_rows(cfg, ll_rows)
        return [([g, H], torch.bfloat16), ([g, K], torch.int64), ([g, K], torch.float32), ([2, g, H], torch.bfloat16),
                ([max(agv_ll_stage_bytes(ll, [H * 2, K * 8, K * 4]), 16)], torch.uint8)]

    def build(self):
        cfg, dev = self.cfg, self.device
        cap, g, H, K, I = max(cfg.per_rank_cap, 1), max(cfg.global_cap, 1), cfg.hidden, cfg.topk, cfg.intermediate
        self.cap = cap
        if self.heap is None:
            self.heap = SymmetricHeap(self.group, required_bytes(self.heap_specs(cfg, self.ll_rows)), dev,
                                      transport=self.transport)
        h = self.heap
        self.agv_h = h.alloc("fx_agv_h", [g, H], torch.bfloat16)
        self.agv_r = h.alloc("fx_agv_r", [g, K], torch.int64)
        self.agv_p = h.alloc("fx_agv_p", [g, K], torch.float32)
        # per-token partial sums of this rank's experts, two copies used alternately layer by layer
        self.partial = h.alloc("fx_partial", [2, g, H], torch.bfloat16)
        self.ll_agv = h.alloc("fx_ll_agv", [max(agv_ll_stage_bytes(self.ll_rows, [H * 2, K * 8, K * 4]), 16)], torch.uint8)
        self.in_hidden = torch.zeros(cap, H, dtype=torch.bfloat16, device=dev)
        self.in_routing = torch.zeros(cap, K, dtype=torch.int64, device=dev)
        self.in_probs = torch.zeros(cap, K, dtype=torch.float32, device=dev)
        self.out_buf = torch.zeros(cap, H, dtype=torch.bfloat16, device=dev)
        self.n_local = torch.zeros(1, dtype=torch.int32, device=dev)
        self.step_metadata = torch.zeros(4, dtype=torch.int32, device=dev)
        self.local_tokens = 0
        E = cfg.num_local_experts
        self.route = RouteBuffers(g, K, E, dev)
        self.act = torch.zeros(max(self.route.max_pairs, 1), I, dtype=torch.bfloat16, device=dev)
        self.y = torch.zeros(max(self.route.max_pairs, 1), H, dtype=torch.bfloat16, device=dev)
        per_layer = E * 3 * H * I * 2
        sets = max(1, min(self.num_layers, int(self.weight_budget_gb * 2**30 // per_layer)))
        self.weights = [ExpertWeights(E, H, I, dev, seed=self.weight_seed * 100003 + s * 1009 + cfg.rank,
                                      layout="packed" if self.layer_kernel else "split")
                        for s in range(sets)]
        st = h.status.view(torch.int32)
        self.meta_plan = MetadataPlan(h, self.n_local, self.step_metadata, cap)
        self.agv_plan = AllGatherVPlan(h, [self.agv_h, self.agv_r, self.agv_p],
                                       [self.in_hidden, self.in_routing, self.in_probs], self.n_local,
                                       self.step_metadata, cap, grid=self.num_sms, threads=self.threads,
                                       ll_stage=self.ll_agv, ll_rows=self.ll_rows)
        self.route_plan = RoutePlan(self.route, self.agv_r.tensor, self.agv_p.tensor, self.step_metadata[0:1],
                                    expert_begin=cfg.rank * E, status=st)
        self.combine_plan = ExpertCombinePlan(h, self.y, self.route, self.partial, self.out_buf, self.n_local,
                                              self.step_metadata, cap, grid=NUM_SMS)
        if self.layer_kernel:
            self.ffn = [ExpertFfnPlan(w, self.route, self.agv_h.tensor, self.act, self.y, st) for w in self.weights]
            self.layer_plan = MoeLayerPlan(h, self.agv_plan, self.route_plan, self.ffn, self.combine_plan, self.meta_plan,
                                           trace=self.phase_trace)
        else:
            self.fc1 = [GroupedGemmPlan(_ext.GEMM_FC1, w.map_gate_up, self.route, self.agv_h.tensor, self.act, 2 * I, H, st)
                        for w in self.weights]
            self.fc2 = [GroupedGemmPlan(_ext.GEMM_FC2, w.map_down, self.route, self.act, self.y, H, I, st)
                        for w in self.weights]
            self.fc2_combine = [Fc2CombinePlan(h, f, self.combine_plan) for f in self.fc2]
            self.dispatch_fc1 = [DispatchRouteFc1Plan(h, self.agv_plan, self.route_plan, f) for f in self.fc1]
        torch.cuda.synchronize()
        dist.barrier(self.group)
        self._built = True

    def setup_batch(self, hidden, topk_idx, topk_weights):
        n = hidden.shape[0]
        if n > self.cap:
            raise ValueError(f"{n} local tokens exceed the per-rank capacity {self.cap}")
        self.local_tokens = n
        if n:
            self.in_hidden[:n].copy_(hidden, non_blocking=True)
            self.in_routing[:n].copy_(topk_idx, non_blocking=True)
            self.in_probs[:n].copy_(topk_weights, non_blocking=True)
        self.n_local.fill_(n)

    @property
    def out(self):
        return self.out_buf[:self.local_tokens]

    def metadata(self):
        self.meta_plan.launch(self.pdl)

    def dispatch(self):
        self.agv_plan.launch(self.pdl)

    def experts(self, layer: int = 0):
        s = layer % len(self.weights)
        self.route_plan.launch(self.pdl)
        if self.layer_kernel:
            self.ffn[s].launch(self.pdl)
        else:
            self.fc1[s].launch(self.pdl)
            self.fc2[s].launch(self.pdl)

    def combine(self):
        self.combine_plan.launch(self.pdl)

    def layer(self, layer: int = 0):
        s = layer % len(self.weights)
        if self.layer_kernel:
            self.layer_plan.launch(s, self.pdl and self.coop_pdl)
            return
        if self.fuse_dispatch:
            self.dispatch_fc1[s].launch(self.pdl and self.coop_pdl)
        else:
            self.dispatch()
            self.route_plan.launch(self.pdl)
            self.fc1[s].launch(self.pdl)
        if self.fuse_combine:
            self.fc2_combine[s].launch(self.pdl and self.coop_pdl)
        else:
            self.fc2[s].launch(self.pdl)
            self.combine()

    def step(self):
        self.layer(0)

    def decode_step(self, num_layers: int):
        if self.layer_kernel:       # one native call: count exchange + one launch per layer
            self.layer_plan.decode_step(num_layers, self.pdl and self.coop_pdl)
            return
        self.metadata()
        for l in range(num_layers):
            self.layer(l)

    def check_health(self):
        self.heap.check_status()

    def _sync_all(self):
        torch.cuda.synchronize()
        dist.barrier(self.group)

    def reference_output(self, hidden, topk_idx, topk_w, layer: int = 0):
        """CPU oracle of one layer for THIS rank's tokens: every expert of every rank (weights
        regenerated from their seeds), fp32 math."""
        cfg = self.cfg
        s = layer % len(self.weights)
        wgu, wd = [], []
        for r in range(cfg.ep_size):
            if r == cfg.rank:
                gu, dn = self.weights[s].w_gate_up, self.weights[s].w_down
            else:   # the same generator calls as ExpertWeights.__init__, with that rank's seed
                g = torch.Generator(device=self.device).manual_seed(self.weight_seed * 100003 + s * 1009 + r)
                E, H, I = cfg.num_local_experts, cfg.hidden, cfg.intermediate
                gu = (torch.randn(E, 2 * I, H, device=self.device, generator=g) * 0.02).to(torch.bfloat16)
                dn = (torch.randn(E, H, I, device=self.device, generator=g) * 0.02).to(torch.bfloat16)
            wgu.append(gu.cpu())
            wd.append(dn.cpu())
        return oracle.moe_layer(hidden.cpu(), topk_idx.cpu(), topk_w.cpu(), torch.cat(wgu), torch.cat(wd))

    def validate(self):
        """One full layer against the CPU oracle at B = 2*ep, at B = 1 (idle ranks) and, when the
        capacity allows, at a realistic batch (up to 4096 tokens over all ranks, multi-block routing,
        every expert busy) where a sample of this rank's tokens is compared."""
        from ..utils.inputs import make_inputs
        cfg, rank = self.cfg, self.cfg.rank
        results = []
        cases = [cfg.ep_size * 2, 1]
        big = min(self.cap * cfg.ep_size, 4096)
        if big > 4 * cfg.ep_size:
            cases.append(big)
        for B in cases:
            counts = self._validation_counts(B)
            if max(counts) > self.cap:
                continue
            h, i, w = make_inputs(cfg, B, self.device, n=counts[rank])
            # The oracle of the previous case takes seconds on the ranks that had tokens and nothing on idle
            # ones: meet on the host first, or the idle ranks' bounded device waits run out.
            self._sync_all()
            self.setup_batch(h, i, w)
            for rep in range(2 if B == big else 1):     # twice at the large batch: counters must come back clean
                self.metadata()
                self.layer(0)
                self._sync_all()
            if counts[rank]:
                n = counts[rank]
                sample = torch.arange(n) if n <= 16 else torch.arange(0, n, max(1, n // 8))[:8]
                ref = self.reference_output(h[sample], i[sample], w[sample])
                got = self.out[sample].float().cpu()
                scale = float(ref.abs().max()) + 1e-6
                err = float((got - ref).abs().max())
                ok = err / scale < 0.05
                detail = (f"n={n} ({sample.numel()} token(s) compared) max|got-ref|={err:.5f} "
                          f"({100 * err / scale:.2f}% of {scale:.4f})")
            else:
                ok, detail = True, "n=0 (idle rank still runs its experts on other ranks' tokens)"
            results.append((f"fused MoE layer vs oracle B={B:<4d}", bool(ok), detail))
        try:
            self.check_health()
        except Exception as e:
            results.append(("fused device status", False, str(e)))
        return results

    def destroy(self):
        if self._own_heap and self.heap is not None:
            self.heap.destroy()
        self.heap = None
        self._built = False
