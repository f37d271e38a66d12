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
    weights = ExpertWeights(E, H, I, DEV, seed=5, std=0.05, layout="split")
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


@pytest.mark.parametrize("T,E,K,H,I,grid", [(64, 16, 4, 256, 128, 148), (37, 4, 2, 1024, 1024, 24), (700, 2, 2, 512, 256, 5),
                                            (3, 8, 2, 256, 128, 148), (4500, 8, 4, 256, 128, 148),
                                            (400, 8, 2, 256, 256, 3), (400, 8, 2, 256, 256, 5)])
def test_expert_ffn_weights_as_m_against_oracle(world1, T, E, K, H, I, grid):
    """The grouped FFN with the weights as the M = 128 operand (gate/up + SwiGLU + down in one
    persistent launch): experts with no token, with a few, and with more than 256 (several passes
    over the same weight block), more units than CTAs, interleaved gate/up rows; about 100 tokens per
    expert (one block per pipeline stage, the next unit's gather indices fetched under the current one)."""
    from moe_comms_benchmarking_b200.ops import oracle
    from moe_comms_benchmarking_b200.ops.experts import ExpertFfnPlan, ExpertWeights, RouteBuffers, RoutePlan
    from moe_comms_benchmarking_b200.parallel.symm_heap import SymmetricHeap
    x, idx, w = _case(T, E, K, H, I, 9)
    if T == 3:
        idx = idx % 3                       # most experts stay empty
        idx[:, 1] = (idx[:, 0] + 1) % 3
    cap = T + 5
    heap = SymmetricHeap(world1, 1 << 20, DEV)
    xs = torch.zeros(cap, H, dtype=torch.bfloat16, device=DEV); xs[:T] = x
    idxs = torch.zeros(cap, K, dtype=torch.int64, device=DEV); idxs[:T] = idx
    ws = torch.zeros(cap, K, device=DEV); ws[:T] = w
    ntok = torch.tensor([T], dtype=torch.int32, device=DEV)
    route = RouteBuffers(cap, K, E, DEV)
    weights = ExpertWeights(E, H, I, DEV, seed=5, std=0.05)
    from moe_comms_benchmarking_b200.ops.experts import pack_weight_tiles
    assert torch.equal(pack_weight_tiles(ExpertWeights.interleave(weights.w_gate_up)), weights.w1)
    act = torch.zeros(route.max_pairs, I, dtype=torch.bfloat16, device=DEV)
    y = torch.zeros(route.max_pairs, H, dtype=torch.bfloat16, device=DEV)
    rp = RoutePlan(route, idxs, ws, ntok, expert_begin=0, status=heap.status, grid=7)
    ffn = ExpertFfnPlan(weights, route, xs, act, y, heap.status, grid=grid)
    for rep in range(2):
        act.fill_(float("nan")); y.fill_(float("nan"))
        rp.launch(); ffn.launch()
        torch.cuda.synchronize()
        heap.check_status()
        off = route.expert_offset.cpu().tolist()
        P = off[E]
        assert P == T * K and int(route.max_rows) == max(off[e + 1] - off[e] for e in range(E))
        ptok, pprob = route.pair_token.cpu(), route.pair_prob.cpu()
        xg = x.cpu().float()[ptok[:P].long()]
        wgu = weights.w_gate_up.cpu().float()
        gu = torch.cat([xg[off[e]:off[e + 1]] @ wgu[e].t() for e in range(E)])
        want_act = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
        got_act = act[:P].float().cpu()
        s = float(want_act.abs().max())
        assert float((got_act - want_act).abs().max()) < 0.02 * s + 1e-3, "gate/up + SwiGLU"
        wd = weights.w_down.cpu().float()
        want_y = torch.cat([got_act[off[e]:off[e + 1]] @ wd[e].t() for e in range(E)]) * pprob[:P].unsqueeze(1)
        got_y = y[:P].float().cpu()
        s = float(want_y.abs().max())
        assert float((got_y - want_y).abs().max()) < 0.02 * s + 1e-3, "down"
        # per-token sum of the pair rows against the full-layer oracle
        pos = route.pair_pos[:T].cpu().long()
        out = got_y[pos.flatten()].view(T, K, H).sum(1)
        ref = oracle.moe_layer(x.cpu(), idx.cpu(), w.cpu(), weights.w_gate_up.cpu(), weights.w_down.cpu())
        assert float((out - ref).abs().max()) < 0.03 * float(ref.abs().max()) + 1e-3, "layer"


@pytest.mark.parametrize("W,B,ll_rows", [(2, 96, 0), (4, 40, 0), (2, 7, 16), (4, 1, 16)])
def test_moe_layer_kernel_emulated_ranks(lib, W, B, ll_rows):
    """The whole-layer kernel (dispatch, routing, experts, combine in one cooperative launch) with W
    ranks emulated on one GPU: the cross-rank protocol of the product kernel against the oracle,
    twice in a row (every counter must come back clean), with an uneven split and packet mode."""
    from moe_comms_benchmarking_b200.ops import _ext, oracle
    from moe_comms_benchmarking_b200.ops.dense import agv_ll_stage_bytes
    from moe_comms_benchmarking_b200.ops.experts import ExpertWeights, RouteBuffers
    from moe_comms_benchmarking_b200.parallel.emulation import EmuWorld
    E_loc, K, H, I = 4, 3, 256, 128
    E = E_loc * W
    counts = [B // W + (1 if r < B % W else 0) for r in range(W)]
    counts[0], counts[-1] = counts[0] + counts[-1] // 2, counts[-1] - counts[-1] // 2     # uneven
    cap, g = max(counts), max(counts) * W
    w = EmuWorld(W, 8 << 20, DEV)
    dst = [w.alloc([g, H], torch.bfloat16), w.alloc([g, K], torch.int64), w.alloc([g, K], torch.float32)]
    partial = w.alloc([2, g, H], torch.bfloat16)
    ll = w.alloc([max(16, agv_ll_stage_bytes(ll_rows, [H * 2, K * 8, K * 4]))], torch.uint8)
    gen = torch.Generator(device=DEV).manual_seed(41)
    ranks = []
    for r in range(W):
        route = RouteBuffers(g, K, E_loc, DEV)
        ranks.append(dict(
            weights=ExpertWeights(E_loc, H, I, DEV, seed=100 + r, std=0.05), route=route, expert_begin=r * E_loc,
            src=(torch.zeros(cap, H, dtype=torch.bfloat16, device=DEV), torch.zeros(cap, K, dtype=torch.int64, device=DEV),
                 torch.zeros(cap, K, device=DEV)),
            dst=tuple(t[r] for t in dst), partial=partial[r], ll_stage=ll[r],
            n_local=torch.tensor([counts[r]], dtype=torch.int32, device=DEV),
            step_meta=torch.zeros(4, dtype=torch.int32, device=DEV),
            act=torch.zeros(route.max_pairs, I, dtype=torch.bfloat16, device=DEV),
            y=torch.zeros(route.max_pairs, H, dtype=torch.bfloat16, device=DEV),
            out=torch.zeros(cap, H, dtype=torch.bfloat16, device=DEV)))
    wgu = torch.cat([d["weights"].w_gate_up.cpu() for d in ranks])
    wd = torch.cat([d["weights"].w_down.cpu() for d in ranks])
    for rep in range(2):
        xs, idxs, ps = [], [], []
        for r, d in enumerate(ranks):
            n = counts[r]
            x = torch.randn(n, H, device=DEV, generator=gen).to(torch.bfloat16)
            idx = torch.stack([torch.randperm(E, device=DEV, generator=gen)[:K] for _ in range(n)]) if n else \
                torch.zeros(0, K, dtype=torch.int64, device=DEV)
            p = torch.rand(n, K, device=DEV, generator=gen) + 0.1
            d["src"][0][:n], d["src"][1][:n], d["src"][2][:n] = x, idx, p
            d["out"].zero_()
            xs.append(x.cpu()); idxs.append(idx.cpu()); ps.append(p.cpu())
        w.metadata([d["n_local"] for d in ranks], [d["step_meta"] for d in ranks], cap)
        w.moe_layer(ranks, grid=148 // W, topk=K, cap=cap, ll_rows=ll_rows)
        w.check_status()
        for r, d in enumerate(ranks):
            ref = oracle.moe_layer(xs[r], idxs[r], ps[r], wgu, wd)
            if counts[r]:
                s = float(ref.abs().max())
                assert float((d["out"][:counts[r]].float().cpu() - ref).abs().max()) < 0.03 * s + 1e-3, f"rank {r} rep {rep}"


def test_fused_dispatcher_routes_more_than_one_block_of_entries(world1):
    """More (token, expert) entries than one block routes alone, so the multi-block routing branch
    (histogram per block, hand-over through the last block, cursors in global memory) runs INSIDE the
    cooperative layer kernel; a sample of tokens is checked against the oracle."""
    from moe_comms_benchmarking_b200.config import Config
    from moe_comms_benchmarking_b200.parallel.fused import FusedExpertDispatcher
    from moe_comms_benchmarking_b200.utils.inputs import make_inputs
    cfg = Config(num_experts=16, topk=8, hidden=256, intermediate=128, ep_size=1, per_rank_cap=2304)
    d = FusedExpertDispatcher(cfg, world1, num_layers=1, weight_budget_gb=0.5)
    d.build()
    h, i, w = make_inputs(cfg, 2304, DEV)          # 18432 entries > 16384
    d.setup_batch(h, i, w)
    for _ in range(2):
        d.decode_step(1)
        torch.cuda.synchronize()
        d.check_health()
    sample = torch.arange(0, 2304, 37)
    ref = d.reference_output(h[sample], i[sample], w[sample])
    s = float(ref.abs().max())
    assert float((d.out[sample].float().cpu() - ref).abs().max()) < 0.05 * s
    d.destroy()


@pytest.mark.parametrize("fuse,fuse_d", [(True, True), (False, False), (True, False), (False, True)])
def test_two_kernel_fused_dispatcher_world1(world1, fuse, fuse_d):
    from moe_comms_benchmarking_b200.config import Config
    from moe_comms_benchmarking_b200.parallel.fused import FusedExpertDispatcher
    from moe_comms_benchmarking_b200.utils.inputs import make_inputs
    from moe_comms_benchmarking_b200.utils.timing import capture_graph
    cfg = Config(num_experts=16, topk=4, hidden=512, intermediate=256, ep_size=1, per_rank_cap=160)
    d = FusedExpertDispatcher(cfg, world1, num_layers=3, weight_budget_gb=1.0, fuse_combine=fuse, fuse_dispatch=fuse_d,
                              layer_kernel=False)
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


def test_layer_kernel_fused_dispatcher_world1(world1):
    from moe_comms_benchmarking_b200.config import Config
    from moe_comms_benchmarking_b200.parallel.fused import FusedExpertDispatcher
    from moe_comms_benchmarking_b200.utils.inputs import make_inputs
    from moe_comms_benchmarking_b200.utils.timing import capture_graph
    cfg = Config(num_experts=16, topk=4, hidden=512, intermediate=256, ep_size=1, per_rank_cap=160)
    d = FusedExpertDispatcher(cfg, world1, num_layers=3, weight_budget_gb=1.0)
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


def test_layer_kernel_phase_trace_world1(world1):
    """The optional device trace of the layer kernel: seven phases in order, none negative, together no
    longer than the step they belong to; and the traced layer still computes the right rows."""
    from moe_comms_benchmarking_b200.config import Config
    from moe_comms_benchmarking_b200.parallel.fused import FusedExpertDispatcher
    from moe_comms_benchmarking_b200.utils.inputs import make_inputs
    cfg = Config(num_experts=16, topk=4, hidden=512, intermediate=256, ep_size=1, per_rank_cap=96)
    d = FusedExpertDispatcher(cfg, world1, num_layers=1, weight_budget_gb=1.0, phase_trace=True)
    d.build()
    h, i, w = make_inputs(cfg, 80, DEV)
    d.setup_batch(h, i, w)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    d.decode_step(1)                       # warm-up
    torch.cuda.synchronize()
    t0.record(); d.decode_step(1); t1.record()
    torch.cuda.synchronize()
    d.check_health()
    phases = d.layer_plan.phase_times()
    assert [n for n, _ in phases] == ["dispatch", "grid barrier", "routing", "grid barrier", "experts", "grid barrier", "combine"]
    assert all(us >= 0 for _, us in phases)
    total = sum(us for _, us in phases)
    assert 0 < total <= t0.elapsed_time(t1) * 1e3 + 50.0
    ref = d.reference_output(h, i, w, layer=0)
    assert float((d.out.float().cpu() - ref).abs().max()) < 0.05 * float(ref.abs().max())
    d.destroy()
