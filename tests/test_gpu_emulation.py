"""Multi-rank protocol of every kernel, emulated on ONE GPU (all ranks inside one cooperative
launch), against the CPU oracle."""
import pytest
import torch

from moe_comms_benchmarking_b200.ops import _ext, oracle
from moe_comms_benchmarking_b200.parallel.emulation import EmuWorld
from moe_comms_benchmarking_b200.parallel.symm_heap import DeviceStatusError

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _scalars(vals):
    return [torch.tensor([v], dtype=torch.int32, device=DEV) for v in vals]


def _metas(world):
    return [torch.zeros(4, dtype=torch.int32, device=DEV) for _ in range(world)]


def test_metadata_two_steps(lib):
    w = EmuWorld(4, 1 << 16, DEV)
    metas = _metas(4)
    for step, counts in enumerate(([3, 0, 5, 2], [1, 1, 0, 7], [0, 0, 0, 0])):
        w.metadata(_scalars(counts), metas, cap=8)
        want = oracle.metadata(counts)
        for r in range(4):
            assert metas[r][:3].tolist() == want[r] and int(metas[r][3]) == step + 1
    w.check_status()


def test_metadata_capacity_error_is_reported(lib):
    w = EmuWorld(2, 1 << 16, DEV)
    w.metadata(_scalars([9, 1]), _metas(2), cap=4)
    with pytest.raises(DeviceStatusError) as e:
        w.check_status()
    assert e.value.code == 2


@pytest.mark.parametrize("grid,threads", [(1, 64), (4, 256), (16, 512)])
def test_all_gather_v_and_reduce_scatter_v(lib, grid, threads):
    W, cap, H, K = 4, 16, 256, 22
    w = EmuWorld(W, 4 << 20, DEV)
    g = torch.Generator(device=DEV).manual_seed(5)
    dst_h = w.alloc([cap * W, H], torch.bfloat16)
    dst_r = w.alloc([cap * W, K], torch.int64)
    dst_p = w.alloc([cap * W, K], torch.float32)       # 88-byte rows: the 8-byte access path
    rsv = w.alloc([cap * W, H], torch.bfloat16)
    rsv32 = w.alloc([cap * W, H], torch.float32)
    metas = _metas(W)
    for counts in ([5, 0, 16, 3], [1, 2, 3, 4]):
        n_locals = _scalars(counts)
        src_h = [torch.randn(cap, H, device=DEV, generator=g).to(torch.bfloat16) for _ in range(W)]
        src_r = [torch.randint(0, 512, (cap, K), device=DEV, generator=g) for _ in range(W)]
        src_p = [torch.rand(cap, K, device=DEV, generator=g) for _ in range(W)]
        w.metadata(n_locals, metas, cap)
        w.all_gather_v([dst_h, dst_r, dst_p], [src_h, src_r, src_p], n_locals, metas, cap, grid, threads)
        valid = sum(counts)
        full_h = oracle.all_gather_v([src_h[r][:counts[r]] for r in range(W)])
        full_r = oracle.all_gather_v([src_r[r][:counts[r]] for r in range(W)])
        full_p = oracle.all_gather_v([src_p[r][:counts[r]] for r in range(W)])
        for r in range(W):
            assert torch.equal(dst_h[r].tensor[:valid], full_h)
            assert torch.equal(dst_r[r].tensor[:valid], full_r)
            assert torch.equal(dst_p[r].tensor[:valid], full_p)
        # reduce-scatter: every rank contributes its own random partial sums
        for buf, dt, tol in ((rsv, torch.bfloat16, 2e-2), (rsv32, torch.float32, 1e-5)):
            for r in range(W):
                buf[r].tensor.copy_(torch.randn(cap * W, H, device=DEV, generator=g).to(dt))
            outs = [torch.zeros(cap, H, dtype=dt, device=DEV) for _ in range(W)]
            w.reduce_scatter_v(outs, buf, n_locals, metas, cap, grid, threads)
            want = oracle.reduce_scatter_v([buf[r].tensor[:valid].cpu() for r in range(W)], counts)
            for r in range(W):
                assert torch.allclose(outs[r][:counts[r]].float().cpu(), want[r], rtol=tol, atol=tol)
    w.check_status()


@pytest.mark.parametrize("grid,threads", [(1, 128), (6, 512)])
def test_low_latency_packet_mode(lib, grid, threads):
    """Small steps travel as flagged packets (no barrier).  Steps alternate between packet mode
    and the ordinary mode (more rows than the limit) on the same buffers."""
    from moe_comms_benchmarking_b200.ops.dense import agv_ll_stage_bytes, rsv_ll_stage_bytes
    W, cap, H, K, LL = 4, 16, 256, 22, 8
    w = EmuWorld(W, 8 << 20, DEV)
    g = torch.Generator(device=DEV).manual_seed(31)
    dst_h = w.alloc([cap * W, H], torch.bfloat16)
    dst_r = w.alloc([cap * W, K], torch.int64)
    dst_p = w.alloc([cap * W, K], torch.float32)
    rsv = w.alloc([cap * W, H], torch.bfloat16)
    st_a = w.alloc([agv_ll_stage_bytes(LL, [H * 2, K * 8, K * 4])], torch.uint8)
    st_r = w.alloc([rsv_ll_stage_bytes(W, LL, cap, H * 2)], torch.uint8)
    metas = _metas(W)
    for counts in ([4, 0, 2, 1], [1, 0, 0, 0], [3, 9, 1, 0], [2, 2, 2, 2], [0, 0, 0, 0], [0, 8, 0, 0], [4, 4, 4, 4]):
        n_locals = _scalars(counts)
        src_h = [torch.randn(cap, H, device=DEV, generator=g).to(torch.bfloat16) for _ in range(W)]
        src_r = [torch.randint(0, 512, (cap, K), device=DEV, generator=g) for _ in range(W)]
        src_p = [torch.rand(cap, K, device=DEV, generator=g) for _ in range(W)]
        for d in (dst_h, dst_r, dst_p):
            for r in range(W):
                d[r].tensor.zero_()
        w.metadata(n_locals, metas, cap)
        w.all_gather_v([dst_h, dst_r, dst_p], [src_h, src_r, src_p], n_locals, metas, cap, grid, threads,
                       ll_stage=st_a, ll_rows=LL)
        valid = sum(counts)
        full = [oracle.all_gather_v([s[r][:counts[r]] for r in range(W)]) for s in (src_h, src_r, src_p)]
        for r in range(W):
            assert torch.equal(dst_h[r].tensor[:valid], full[0])
            assert torch.equal(dst_r[r].tensor[:valid], full[1])
            assert torch.equal(dst_p[r].tensor[:valid], full[2])
        for r in range(W):
            rsv[r].tensor.copy_(torch.randn(cap * W, H, device=DEV, generator=g).to(torch.bfloat16))
        outs = [torch.zeros(cap, H, dtype=torch.bfloat16, device=DEV) for _ in range(W)]
        w.reduce_scatter_v(outs, rsv, n_locals, metas, cap, grid, threads, ll_stage=st_r, ll_rows=LL)
        want = oracle.reduce_scatter_v([rsv[r].tensor[:valid].cpu() for r in range(W)], counts)
        for r in range(W):
            assert torch.allclose(outs[r][:counts[r]].float().cpu(), want[r], rtol=2e-2, atol=2e-2)
    w.check_status()


def _a2a_case(W, E, K, H, counts, fp8, seed):
    cap = max(max(counts), 1)
    w = EmuWorld(W, 16 << 20, DEV)
    g = torch.Generator(device=DEV).manual_seed(seed)
    b = w.a2a_buffers(cap, H, K, fp8)
    xs = [torch.randn(cap, H, device=DEV, generator=g).to(torch.bfloat16) for _ in range(W)]
    idxs = [torch.stack([torch.randperm(E, device=DEV, generator=g)[:K] for _ in range(cap)]) for _ in range(W)]
    ws = [torch.rand(cap, K, device=DEV, generator=g) for _ in range(W)]
    return w, b, xs, idxs, ws, _scalars(counts), cap


@pytest.mark.parametrize("counts", [[5, 0, 8, 3], [1, 0, 0, 0], [0, 0, 0, 0]])
def test_a2a_dispatch_and_combine_bf16(lib, counts):
    W, E, K, H = 4, 32, 6, 256
    w, b, xs, idxs, ws, n_locals, cap = _a2a_case(W, E, K, H, counts, False, 11)
    outs = [torch.zeros(cap, H, dtype=torch.bfloat16, device=DEV) for _ in range(W)]
    for _ in range(2):      # twice: counters and epochs must return to a clean state
        w.a2a_dispatch(b, xs, idxs, ws, n_locals, E)
        recv = oracle.a2a_dispatch([xs[r][:counts[r]].cpu() for r in range(W)],
                                   [idxs[r][:counts[r]].cpu() for r in range(W)], E, W)
        for d in range(W):
            got_counts = b["recv_count"][d].tensor[:W].tolist()
            assert got_counts == [recv[d][s][0].numel() for s in range(W)]
            for s in range(W):
                c = got_counts[s]
                if not c:
                    continue
                src_tok = b["recv_src"][d].tensor[s, :c].cpu().long()
                order = torch.argsort(src_tok)
                assert torch.equal(src_tok[order], recv[d][s][0])
                assert torch.equal(b["recv_x"][d].tensor[s, :c].cpu()[order], recv[d][s][1])
                assert torch.equal(b["recv_idx"][d].tensor[s, :c].cpu()[order], idxs[s][:counts[s]].cpu()[recv[d][s][0]])
                assert torch.equal(b["recv_w"][d].tensor[s, :c].cpu()[order], ws[s][:counts[s]].cpu()[recv[d][s][0]])
        w.a2a_combine(b, outs, n_locals)
        for r in range(W):
            ref = oracle.roundtrip_identity(xs[r][:counts[r]], idxs[r][:counts[r]].cpu(), E, W)
            assert torch.allclose(outs[r][:counts[r]].float().cpu(), ref, rtol=2e-2, atol=2e-2)
    w.check_status()


def test_launch_numbers_do_not_depend_on_the_grid(lib):
    """The launch number that the all-to-all combine hands from block 0 to the other blocks, and the
    packet flag of the low-latency collectives, are per-block counters that the host levels when the
    grid of a site changes: a launch with more blocks than any earlier one must neither skip the
    combine's leading cross-rank barrier nor disagree about the flag.  Every launch uses new data,
    so a block that ran ahead of the barrier or matched a stale packet produces a wrong result."""
    W, E, K, H, counts = 4, 32, 6, 256, [5, 2, 8, 3]
    w, b, xs, idxs, ws, n_locals, cap = _a2a_case(W, E, K, H, counts, False, 19)
    outs = [torch.zeros(cap, H, dtype=torch.bfloat16, device=DEV) for _ in range(W)]
    g = torch.Generator(device=DEV).manual_seed(3)
    for grid in (2, 8, 16, 3, 16):
        xs = [torch.randn(cap, H, device=DEV, generator=g).to(torch.bfloat16) for _ in range(W)]
        w.a2a_dispatch(b, xs, idxs, ws, n_locals, E, grid=grid)
        w.a2a_combine(b, outs, n_locals, grid=grid)
        for r in range(W):
            ref = oracle.roundtrip_identity(xs[r][:counts[r]], idxs[r][:counts[r]].cpu(), E, W)
            assert torch.allclose(outs[r][:counts[r]].float().cpu(), ref, rtol=2e-2, atol=2e-2)
    w.check_status()
    # packet mode of the stand-alone all-gather / reduce-scatter with a changing grid
    from moe_comms_benchmarking_b200.ops.dense import agv_ll_stage_bytes, rsv_ll_stage_bytes
    cap, LL = 8, 8
    w = EmuWorld(W, 8 << 20, DEV)
    dst = w.alloc([cap * W, H], torch.bfloat16)
    rsv = w.alloc([cap * W, H], torch.bfloat16)
    st_a = w.alloc([agv_ll_stage_bytes(LL, [H * 2])], torch.uint8)
    st_r = w.alloc([rsv_ll_stage_bytes(W, LL, cap, H * 2)], torch.uint8)
    metas, counts = _metas(W), [2, 1, 0, 3]
    n_locals = _scalars(counts)
    for grid in (1, 6, 2, 12):
        src = [torch.randn(cap, H, device=DEV, generator=g).to(torch.bfloat16) for _ in range(W)]
        w.metadata(n_locals, metas, cap)
        w.all_gather_v([dst], [src], n_locals, metas, cap, grid, 128, ll_stage=st_a, ll_rows=LL)
        full = oracle.all_gather_v([src[r][:counts[r]] for r in range(W)])
        for r in range(W):
            assert torch.equal(dst[r].tensor[:sum(counts)], full)
            rsv[r].tensor.copy_(torch.randn(cap * W, H, device=DEV, generator=g).to(torch.bfloat16))
        outs = [torch.zeros(cap, H, dtype=torch.bfloat16, device=DEV) for _ in range(W)]
        w.reduce_scatter_v(outs, rsv, n_locals, metas, cap, grid, 128, ll_stage=st_r, ll_rows=LL)
        want = oracle.reduce_scatter_v([rsv[r].tensor[:sum(counts)].cpu() for r in range(W)], counts)
        for r in range(W):
            assert torch.allclose(outs[r][:counts[r]].float().cpu(), want[r], rtol=2e-2, atol=2e-2)
    w.check_status()


@pytest.mark.parametrize("ll_rows", [0, 20])
@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("grid,threads", [(1, 64), (6, 256)])
def test_a2a_step_kernel(lib, fp8, grid, threads, ll_rows):
    """The persistent all-to-all step (count exchange + every layer in one launch): token-indexed
    slots, packed metadata rows with the layer's stamp, one barrier per layer; steps of 1-5 layers with
    idle ranks; received rows / routing / stamps and the combined rows against the oracle.  With
    ``ll_rows`` the small steps run in packet mode (flagged packets, credits, no barrier) and the step of 48
    tokens on the barrier path, in the same sequence of launches."""
    W, E, K, H, cap = 4, 32, 6, 512, 12
    w = EmuWorld(W, 16 << 20, DEV)
    b = w.a2a_step_buffers(cap, H, K, fp8, ll_rows=ll_rows)
    g = torch.Generator(device=DEV).manual_seed(29)
    metas = [torch.zeros(8, dtype=torch.int32, device=DEV) for _ in range(W)]
    outs = [torch.zeros(cap, H, dtype=torch.bfloat16, device=DEV) for _ in range(W)]
    epr = E // W
    if fp8:
        for r in range(W):
            b["y"][r].tensor.copy_(torch.randn(2, W, cap, H, device=DEV, generator=g))
    for counts, layers in (([5, 0, 12, 3], 5), ([1, 0, 0, 0], 2), ([0, 0, 0, 0], 1), ([12, 12, 12, 12], 2), ([2, 7, 1, 4], 1),
                           ([3, 3, 3, 3], 4)):
        xs = [torch.randn(cap, H, device=DEV, generator=g).to(torch.bfloat16) for _ in range(W)]
        idxs = [torch.stack([torch.randperm(E, device=DEV, generator=g)[:K] for _ in range(cap)]) for _ in range(W)]
        ws = [torch.rand(cap, K, device=DEV, generator=g) for _ in range(W)]
        if fp8:
            xs[0][0, :128] = 0
        for o in outs:
            o.fill_(-7.0)
        w.a2a_step(b, xs, idxs, ws, outs, _scalars(counts), metas, E, layers, grid=grid, threads=threads)
        par, stamp = int(metas[0][5]), int(metas[0][7])
        assert metas[0][:3].tolist() == oracle.metadata(counts)[0]
        assert int(metas[0][6]) == int(0 < sum(counts) <= ll_rows)
        for d in range(W):
            for s in range(W):
                c = counts[s]
                if not c:
                    continue
                words = b["recv_meta"][d].tensor[par, s, :c].view(torch.int32).view(c, -1)
                here = ((idxs[s][:c] // epr) == d).any(dim=1)
                assert torch.equal(words[:, 0] == stamp, here)
                sel = here.nonzero().flatten()
                if not sel.numel():
                    continue
                assert torch.equal(words[sel, 1].long(), sel)
                assert torch.equal(words[sel][:, 2:2 + 2 * K:2].long(), idxs[s][sel])
                assert torch.equal(words[sel][:, 3:3 + 2 * K:2].contiguous().view(torch.float32), ws[s][sel])
                if fp8:
                    q = b["recv_x"][d].tensor[par, s][sel].cpu().view(torch.float8_e4m3fn)
                    sc = b["recv_scale"][d].tensor[par, s][sel].cpu()
                    want = xs[s][sel].float().cpu()
                    _, s_ref = oracle.quant_e4m3_1x128(want)
                    assert torch.allclose(sc, s_ref, rtol=1e-6, atol=0)
                    back = oracle.dequant_e4m3_1x128(q, sc)
                    assert ((back - want).abs() <= 0.0625 * want.abs() + 2e-3 * sc.repeat_interleave(128, dim=1)).all()
                else:
                    assert torch.equal(b["recv_x"][d].tensor[par, s][sel], xs[s][sel])
        for r in range(W):
            c = counts[r]
            if not c:
                continue
            if not fp8:         # identity expert: the combine reads the received rows
                ref = oracle.roundtrip_identity(xs[r][:c], idxs[r][:c].cpu(), E, W)
            else:               # the sum of one expert-output row per distinct destination rank
                ref = torch.zeros(c, H)
                for d in range(W):
                    here = ((idxs[r][:c] // epr) == d).any(dim=1).cpu()
                    ref += b["y"][d].tensor[par, r, :c].float().cpu() * here[:, None]
            assert torch.allclose(outs[r][:c].float().cpu(), ref, rtol=2e-2, atol=2e-2)
    w.check_status()


def test_a2a_fp8_dispatch(lib):
    W, E, K, H, counts = 2, 16, 4, 512, [6, 3]
    w, b, xs, idxs, ws, n_locals, cap = _a2a_case(W, E, K, H, counts, True, 13)
    xs[0][0, :128] = 0      # an all-zero block must get scale 1 and zero values
    w.a2a_dispatch(b, xs, idxs, ws, n_locals, E)
    recv = oracle.a2a_dispatch([xs[r][:counts[r]].cpu() for r in range(W)],
                               [idxs[r][:counts[r]].cpu() for r in range(W)], E, W)
    for d in range(W):
        for s in range(W):
            c = int(b["recv_count"][d].tensor[s])
            assert c == recv[d][s][0].numel()
            if not c:
                continue
            order = torch.argsort(b["recv_src"][d].tensor[s, :c].cpu().long())
            q = b["recv_x"][d].tensor[s, :c].cpu()[order].view(torch.float8_e4m3fn)
            sc = b["recv_scale"][d].tensor[s, :c].cpu()[order]
            want = recv[d][s][1].float()
            q_ref, s_ref = oracle.quant_e4m3_1x128(want)
            assert torch.allclose(sc, s_ref, rtol=1e-6, atol=0)
            back = oracle.dequant_e4m3_1x128(q, sc)
            assert ((back - want).abs() <= 0.0625 * want.abs() + 2e-3 * sc.repeat_interleave(128, dim=1)).all()
            assert (q.float() == q_ref.float()).float().mean() > 0.999
    w.check_status()


def test_a2a_bad_expert_id_is_reported(lib):
    W, E, K, H = 2, 16, 4, 256
    w, b, xs, idxs, ws, n_locals, cap = _a2a_case(W, E, K, H, [2, 2], False, 17)
    idxs[1][0, 0] = 99
    w.a2a_dispatch(b, xs, idxs, ws, n_locals, E)
    with pytest.raises(DeviceStatusError) as e:
        w.check_status()
    assert e.value.code == 4


@pytest.mark.parametrize("hidden", [256, 1024, 4096])
def test_rs_add_norm_ag(lib, hidden):
    W, tokens = 2, 8
    w = EmuWorld(W, 1 << 20, DEV)
    g = torch.Generator(device=DEV).manual_seed(23)
    buf = w.alloc([tokens, hidden], torch.bfloat16)
    parts = [torch.randn(tokens, hidden, device=DEV, generator=g).to(torch.bfloat16) for _ in range(W)]
    res = [torch.randn(tokens // W, hidden, device=DEV, generator=g).to(torch.bfloat16) for _ in range(W)]
    weight = (1 + 0.1 * torch.randn(hidden, device=DEV, generator=g)).to(torch.bfloat16)
    for r in range(W):
        buf[r].tensor.copy_(parts[r])
    want, want_res = oracle.rs_add_norm_ag([p.cpu() for p in parts], [r_.cpu() for r_ in res], weight.cpu(), 1e-5)
    w.rs_add_norm_ag(buf, res, weight, 1e-5, grid=3)
    for r in range(W):
        assert torch.allclose(buf[r].tensor.float().cpu(), want, rtol=2e-2, atol=2e-2)
        assert torch.allclose(res[r].float().cpu(), want_res[r].float(), rtol=2e-2, atol=2e-2)
    w.check_status()


def test_barrier_rounds_and_bounded_wait(lib):
    """A healthy barrier passes many rounds.  With a rank that never arrives the wait runs out:
    the kernel returns, the status word says timeout, and the context keeps working."""
    w = EmuWorld(4, 1 << 16, DEV)
    w.barrier_test(grid=8, rounds=50)
    w.check_status()
    assert int(w.epochs[0][_ext.SITE_TEST * _ext.MAX_BLOCKS]) == 50
    lonely = EmuWorld(2, 1 << 16, DEV, timeout_s=0.05, phantom_ranks=1)
    lonely.barrier_test(grid=2, rounds=1)
    with pytest.raises(DeviceStatusError) as e:
        lonely.check_status()
    assert e.value.code == 1 and e.value.words[1] == _ext.SITE_TEST and e.value.words[4] == 3
    x = torch.ones(8, device=DEV)
    assert float((x * 2).sum()) == 16.0          # the context is still usable
    w.barrier_test(grid=8, rounds=1)
    w.check_status()
