"""Expert path on one GPU: routing kernel, tcgen05 grouped GEMMs (FC1 with fused token gather and
SwiGLU, FC2 with routing-weight epilogue) and the combine, each against the fp32 CPU oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(T, E, K, H, I, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    x = torch.randn(T, H, device=DEV, generator=g).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(E, device=DEV, generator=g)[:K] for _ in range(T)])
    w = torch.rand(T, K, device=DEV, generator=g) + 0.1
    return x, idx, w


@pytest.mark.parametrize("T,E,K,H,I", [(200, 8, 4, 256, 128), (37, 4, 2, 1024, 1024), (300, 2, 2, 512, 256),
                                       (4500, 8, 4, 256, 128)])
def test_route_fc1_fc2_combine_against_oracle(world1, T, E, K, H, I):
    from moe_comms_benchmarking_b200.ops import _ext, oracle
    from moe_comms_benchmarking_b200.ops.experts import (ExpertCombinePlan, ExpertWeights, GroupedGemmPlan, RouteBuffers,
                                                         RoutePlan)
    from moe_comms_benchmarking_b200.parallel.symm_heap import SymmetricHeap
    x, idx, w = _case(T, E, K, H, I, 3)
    cap = T + 5
    heap = SymmetricHeap(world1, cap * H * 2 + (1 << 20), DEV)
    partial = heap.alloc("partial", [cap, H], torch.bfloat16)
    status = heap.status
    xs = torch.zeros(cap, H, dtype=torch.bfloat16, device=DEV); xs[:T] = x
    idxs = torch.zeros(cap, K, dtype=torch.int64, device=DEV); idxs[:T] = idx
    ws = torch.zeros(cap, K, device=DEV); ws[:T] = w
    ntok = torch.tensor([T], dtype=torch.int32, device=DEV)
    meta = torch.tensor([T, 0, T, 1], dtype=torch.int32, device=DEV)
    route = RouteBuffers(cap, K, E, DEV)
    weights = ExpertWeights(E, H, I, DEV, seed=5, std=0.05)
    act = torch.zeros(route.max_pairs, I, dtype=torch.bfloat16, device=DEV)
    y = torch.zeros(route.max_pairs, H, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(cap, H, dtype=torch.bfloat16, device=DEV)
    rp = RoutePlan(route, idxs, ws, ntok, expert_begin=0, status=status, grid=7)
    fc1 = GroupedGemmPlan(_ext.GEMM_FC1, weights.map_gate_up, route, xs, act, 2 * I, H, status, grid=5)
    fc2 = GroupedGemmPlan(_ext.GEMM_FC2, weights.map_down, route, act, y, H, I, status, grid=148)
    comb = ExpertCombinePlan(heap, y, route, partial, out, ntok, meta, cap, grid=16, threads=256)
    for rep in range(2):        # twice: scratch counters must come back clean
        rp.launch(); fc1.launch(); fc2.launch(); comb.launch()
        torch.cuda.synchronize()
        heap.check_status()
        # routing: per-expert segments hold exactly the tokens routed to that expert
        off = route.expert_offset.cpu().tolist()
        ptok, pprob, ppos = route.pair_token.cpu(), route.pair_prob.cpu(), route.pair_pos.cpu()
        assert off[E] == T * K
        ntiles = int(route.num_m_tiles)
        assert ntiles == sum((off[e + 1] - off[e] + 127) // 128 for e in range(E))
        for e in range(E):
            want = (idx.cpu() == e).any(dim=1).nonzero().flatten().tolist()
            assert sorted(ptok[off[e]:off[e + 1]].tolist()) == want
        tt, kk = torch.arange(T).repeat_interleave(K), torch.arange(K).repeat(T)
        pos = ppos[:T].flatten().long()
        assert (pos >= 0).all() and torch.equal(ptok[pos].long(), tt)
        assert torch.equal(pprob[pos], w.cpu().flatten())
        pair_expert = torch.bucketize(pos, torch.tensor(off[1:]), right=True)
        assert torch.equal(pair_expert, idx.cpu().flatten())
        # FC1: act rows against silu(x Wg^T) * (x Wu^T)
        P = off[E]
        pe = torch.bucketize(torch.arange(P), torch.tensor(off[1:]), right=True)
        xg = x.cpu().float()[ptok[:P].long()]
        wgu = weights.w_gate_up.cpu().float()
        gu = torch.cat([xg[off[e]:off[e + 1]] @ wgu[e].t() for e in range(E)])
        want_act = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
        got_act = act[:P].float().cpu()
        s = float(want_act.abs().max())
        assert float((got_act - want_act).abs().max()) < 0.02 * s + 1e-3, "FC1"
        # FC2 on the kernel's own bf16 activations
        wd = weights.w_down.cpu().float()
        want_y = torch.cat([got_act[off[e]:off[e + 1]] @ wd[e].t() for e in range(E)]) * pprob[:P].unsqueeze(1)
        got_y = y[:P].float().cpu()
        s = float(want_y.abs().max())
        assert float((got_y - want_y).abs().max()) < 0.02 * s + 1e-3, "FC2"
        # whole layer against the oracle
        ref = oracle.moe_layer(x.cpu(), idx.cpu(), w.cpu(), weights.w_gate_up.cpu(), weights.w_down.cpu())
        s = float(ref.abs().max())
        assert float((out[:T].float().cpu() - ref).abs().max()) < 0.03 * s + 1e-3, "layer"


@pytest.mark.parametrize("fuse,fuse_d", [(True, True), (False, False), (True, False), (False, True)])
def test_fused_dispatcher_world1(world1, fuse, fuse_d):
    from moe_comms_benchmarking_b200.config import Config
    from moe_comms_benchmarking_b200.parallel.fused import FusedExpertDispatcher
    from moe_comms_benchmarking_b200.utils.inputs import make_inputs
    from moe_comms_benchmarking_b200.utils.timing import capture_graph
    cfg = Config(num_experts=16, topk=4, hidden=512, intermediate=256, ep_size=1, per_rank_cap=160)
    d = FusedExpertDispatcher(cfg, world1, num_layers=3, weight_budget_gb=1.0, fuse_combine=fuse, fuse_dispatch=fuse_d)
    d.build()
    for name, ok, detail in d.validate():
        assert ok, f"{name}: {detail}"
    h, i, w = make_inputs(cfg, 150, DEV)
    d.setup_batch(h, i, w)
    g = capture_graph(lambda: d.decode_step(3))
    g.replay()
    torch.cuda.synchronize()
    d.check_health()
    ref = d.reference_output(h, i, w, layer=2)
    s = float(ref.abs().max())
    assert float((d.out.float().cpu() - ref).abs().max()) < 0.05 * s
    d.destroy()
