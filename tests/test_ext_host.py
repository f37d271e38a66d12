"""Library build, struct layouts and host-side argument validation (CPU: nothing is launched)."""
import ctypes as C

import pytest
import torch

from moe_comms_benchmarking_b200.ops import _ext
from moe_comms_benchmarking_b200.ops.a2a import A2ABuffers, A2ACombinePlan, A2ADispatchPlan
from moe_comms_benchmarking_b200.ops.dense import AllGatherVPlan, MetadataPlan, ReduceScatterVPlan
from moe_comms_benchmarking_b200.ops.norm import RsAddNormAgPlan
from moe_comms_benchmarking_b200.parallel.symm_heap import (RESERVED_BYTES, DeviceStatusError, SymmetricHeap,
                                                            SymmetricHeapManager, required_bytes)


def test_library_builds_and_layouts_match(lib):
    assert lib.mcb_max_ranks() == _ext.MAX_RANKS
    assert lib.mcb_max_blocks() == _ext.MAX_BLOCKS
    assert lib.mcb_num_sites() == _ext.NUM_SITES
    assert lib.mcb_sizeof_ctx() == C.sizeof(_ext.McbCtx)


def _heap(nbytes=1 << 20):
    return SymmetricHeap(None, nbytes, "cpu")


def test_heap_bump_allocator_and_registry():
    h = _heap()
    a = h.alloc("a", [10, 3], torch.float32)
    b = h.alloc("b", [7], torch.int64)
    assert a.offset == RESERVED_BYTES and a.offset % 256 == 0 and b.offset % 256 == 0
    assert b.offset >= a.offset + a.nbytes
    assert h.alloc("a", [10, 3], torch.float32) is a
    with pytest.raises(ValueError):
        h.alloc("a", [11, 3], torch.float32)
    with pytest.raises(MemoryError):
        h.alloc("huge", [1 << 22], torch.float32)
    a.tensor.fill_(3.0)
    assert h.buffer[a.offset:a.offset + 4].view(torch.float32).item() == 3.0
    assert required_bytes([([10, 3], torch.float32), ([7], torch.int64)]) == RESERVED_BYTES + 256 + 256
    c = h.ctx()
    assert c.world == 1 and c.rank == 0 and c.transport == _ext.TRANSPORT_P2P
    assert c.heap_peer[0] == c.heap_local == h.buffer.data_ptr()


def test_heap_manager_registry():
    SymmetricHeapManager.destroy()
    assert not SymmetricHeapManager.is_initialized("k")
    h = SymmetricHeapManager.get_heap("k", None, 1 << 16, device="cpu")
    assert SymmetricHeapManager.get_heap("k") is h and SymmetricHeapManager.is_initialized("k")
    SymmetricHeapManager.destroy("k")
    assert not SymmetricHeapManager.is_initialized("k")


def test_multimem_transport_needs_multicast():
    with pytest.raises(RuntimeError):
        SymmetricHeap(None, 1 << 16, "cpu", transport="multimem")


def test_heap_allocator_choice(monkeypatch):
    """The allocator is a named choice (argument first, then the environment); a CPU heap or a world of one
    needs none of them, whatever is asked for."""
    with pytest.raises(ValueError):
        SymmetricHeap(None, 1 << 16, "cpu", allocator="cudamalloc")
    h = SymmetricHeap(None, 1 << 16, "cpu", allocator="native")
    assert h.allocator == "native" and h.buffer.device.type == "cpu" and h.mc_ptr == 0
    monkeypatch.setenv("MCB_HEAP_ALLOCATOR", "native")
    assert SymmetricHeap(None, 1 << 16, "cpu").allocator == "native"
    monkeypatch.delenv("MCB_HEAP_ALLOCATOR")
    assert SymmetricHeap(None, 1 << 16, "cpu").allocator == "torch"


def test_status_error_decoding():
    e = DeviceStatusError([1, 2, 7, 5, 8, 3, 0, 0])
    assert e.code == 1 and "timeout" in str(e) and "site 2 block 7 on rank 3" in str(e)


def test_dense_plans_validate_arguments():
    h = _heap(4 << 20)
    cap, H, K = 8, 64, 6
    n_local = torch.zeros(1, dtype=torch.int32)
    meta = torch.zeros(4, dtype=torch.int32)
    gh = h.alloc("gh", [cap, H], torch.bfloat16)
    gr = h.alloc("gr", [cap, K], torch.int64)
    src_h = torch.zeros(cap, H, dtype=torch.bfloat16)
    src_r = torch.zeros(cap, K, dtype=torch.int64)
    MetadataPlan(h, n_local, meta, cap)
    with pytest.raises(ValueError):
        MetadataPlan(h, torch.zeros(1, dtype=torch.int64), meta, cap)
    AllGatherVPlan(h, [gh, gr], [src_h, src_r], n_local, meta, cap)
    with pytest.raises(ValueError):      # source smaller than capacity
        AllGatherVPlan(h, [gh], [src_h[:4]], n_local, meta, cap)
    with pytest.raises(ValueError):      # gathered buffer too small
        AllGatherVPlan(h, [gh], [src_h], n_local, meta, cap * 2)
    with pytest.raises(ValueError):      # dtype mismatch
        AllGatherVPlan(h, [gh], [src_h.float()], n_local, meta, cap)
    with pytest.raises(ValueError):      # row not a multiple of 4 bytes
        odd = h.alloc("odd", [cap, 3], torch.uint8)
        AllGatherVPlan(h, [odd], [torch.zeros(cap, 3, dtype=torch.uint8)], n_local, meta, cap)
    with pytest.raises(ValueError):      # grid beyond the flag slots
        AllGatherVPlan(h, [gh], [src_h], n_local, meta, cap, grid=_ext.MAX_BLOCKS + 1)
    out = torch.zeros(cap, H, dtype=torch.bfloat16)
    ReduceScatterVPlan(h, out, gh, n_local, meta, cap)
    with pytest.raises(ValueError):      # rows must be multiples of 16 bytes
        g6 = h.alloc("g6", [cap, 6], torch.bfloat16)
        ReduceScatterVPlan(h, torch.zeros(cap, 6, dtype=torch.bfloat16), g6, n_local, meta, cap)
    with pytest.raises(ValueError):
        ReduceScatterVPlan(h, out.float(), gh, n_local, meta, cap)


def test_a2a_and_norm_plans_validate_arguments():
    h = _heap(8 << 20)
    cap, H, K = 4, 256, 4
    bufs = A2ABuffers(h, cap, H, K, fp8=False)
    assert bufs.y is bufs.recv_x
    n_local = torch.zeros(1, dtype=torch.int32)
    x = torch.zeros(cap, H, dtype=torch.bfloat16)
    idx = torch.zeros(cap, K, dtype=torch.int64)
    w = torch.ones(cap, K)
    A2ADispatchPlan(h, bufs, x, idx, w, n_local, 16)
    with pytest.raises(ValueError):
        A2ADispatchPlan(h, bufs, x.float(), idx, w, n_local, 16)
    with pytest.raises(ValueError):
        A2ADispatchPlan(h, bufs, x, idx.int(), w, n_local, 16)
    A2ACombinePlan(h, bufs, torch.zeros(cap, H, dtype=torch.bfloat16), n_local)
    with pytest.raises(ValueError):
        A2ABuffers(h, cap, 200, K, fp8=True, prefix="bad")
    b8 = A2ABuffers(h, cap, H, K, fp8=True, prefix="f8")
    assert b8.recv_scale.tensor.shape == (1, cap, 2) and b8.y is not b8.recv_x
    buf = h.alloc("norm", [8, 64], torch.bfloat16)
    RsAddNormAgPlan(h, buf, torch.zeros(8, 64, dtype=torch.bfloat16), torch.ones(64, dtype=torch.bfloat16))
    with pytest.raises(ValueError):
        RsAddNormAgPlan(h, buf, torch.zeros(4, 64, dtype=torch.bfloat16), torch.ones(64, dtype=torch.bfloat16))


def test_expert_plans_validate_arguments(lib):
    from moe_comms_benchmarking_b200.ops.experts import (DispatchRouteFc1Plan, ExpertCombinePlan, Fc2CombinePlan,
                                                         GroupedGemmPlan, RouteBuffers, RoutePlan)
    h = _heap(8 << 20)
    T, K, E, H, I = 16, 4, 8, 256, 128
    route = RouteBuffers(T, K, E, "cpu")
    assert route.max_pairs == T * 4 and route.max_tiles == E + route.max_pairs // 128 + 1
    idx = torch.zeros(T, K, dtype=torch.int64)
    ntok = torch.zeros(1, dtype=torch.int32)
    rp = RoutePlan(route, idx, None, ntok, expert_begin=0)
    with pytest.raises(ValueError):
        RoutePlan(route, idx.int(), None, ntok, expert_begin=0)
    with pytest.raises(ValueError):
        RoutePlan(route, idx, None, ntok, expert_begin=0, grid=500)
    x = torch.zeros(T, H, dtype=torch.bfloat16)
    act = torch.zeros(route.max_pairs, I, dtype=torch.bfloat16)
    y = torch.zeros(route.max_pairs, H, dtype=torch.bfloat16)
    tmap = (None, 0)            # plans only store the tensor-map handle
    fc1 = GroupedGemmPlan(_ext.GEMM_FC1, tmap, route, x, act, 2 * I, H)
    fc2 = GroupedGemmPlan(_ext.GEMM_FC2, tmap, route, act, y, H, I)
    with pytest.raises(ValueError):      # A rows do not match k_total
        GroupedGemmPlan(_ext.GEMM_FC1, tmap, route, x, act, 2 * I, H * 2)
    with pytest.raises(ValueError):      # out has the wrong width
        GroupedGemmPlan(_ext.GEMM_FC2, tmap, route, act, act, H, I)
    with pytest.raises(ValueError):      # k_total not a multiple of 64
        GroupedGemmPlan(_ext.GEMM_FC2, tmap, route, torch.zeros(route.max_pairs, 96, dtype=torch.bfloat16), y, H, 96)
    partial = h.alloc("partial", [T, H], torch.bfloat16)
    meta = torch.zeros(4, dtype=torch.int32)
    out = torch.zeros(T, H, dtype=torch.bfloat16)
    comb = ExpertCombinePlan(h, y, route, partial, out, ntok, meta, T)
    with pytest.raises(ValueError):      # partial buffer smaller than the capacity
        ExpertCombinePlan(h, y, route, partial, out, ntok, meta, T * 2)
    Fc2CombinePlan(h, fc2, comb)
    with pytest.raises(ValueError):
        Fc2CombinePlan(h, fc1, comb)
    with pytest.raises(ValueError):      # all blocks must be resident at once
        Fc2CombinePlan(h, fc2, comb, grid=149)
    gh = h.alloc("gh2", [T, H], torch.bfloat16)
    agv = AllGatherVPlan(h, [gh], [x], ntok, meta, T)
    DispatchRouteFc1Plan(h, agv, rp, fc1)
    with pytest.raises(ValueError):
        DispatchRouteFc1Plan(h, agv, rp, fc2)


def test_capability_checks():
    from moe_comms_benchmarking_b200 import ops
    assert not ops.is_device_multimem_capable("cpu") and not ops.is_device_tcgen05_capable("cpu")
    h = _heap(1 << 16)
    assert not ops.heap_has_multicast(h)
    assert ops.row_access_bytes(torch.zeros(4, 1024, dtype=torch.bfloat16)) == 16
    assert ops.row_access_bytes(torch.zeros(4, 22, dtype=torch.float32)) == 8      # 88-byte rows
    assert ops.row_access_bytes(torch.zeros(4, 3, dtype=torch.float32)) == 4
    assert ops.row_access_bytes(torch.zeros(4, 3, dtype=torch.uint8)) == 0
    assert ops.row_access_bytes(torch.zeros(4, 8, dtype=torch.float32).t()) == 0   # not contiguous
    assert ops.are_tensors_gather_eligible(torch.zeros(2, 22, dtype=torch.int64), torch.zeros(2, 22))
    assert not ops.are_tensors_gather_eligible()
    assert ops.are_tensors_reduce_eligible(torch.zeros(2, 1024, dtype=torch.bfloat16))
    assert not ops.are_tensors_reduce_eligible(torch.zeros(2, 22))                 # 88-byte rows
    assert not ops.are_tensors_reduce_eligible(torch.zeros(2, 8, dtype=torch.int32))


def test_step_plans_validate_arguments():
    """Host-side checks of the persistent step plans (dense and all-to-all): shapes, capacities,
    parity buffers, packet staging, fp8 tensor layout.  Nothing is launched."""
    from moe_comms_benchmarking_b200.ops.a2a import A2AStepBuffers, A2AStepPlan, a2a_meta_row_bytes
    from moe_comms_benchmarking_b200.ops.dense import (DenseStepPlan, agv_ll_stage_bytes, rsv_ll_stage_bytes,
                                                       step_credit_bytes)
    h = _heap(16 << 20)
    cap, H, K = 8, 256, 6
    n_local = torch.zeros(1, dtype=torch.int32)
    meta8 = torch.zeros(8, dtype=torch.int32)
    g2h = h.alloc("g2h", [2, cap, H], torch.bfloat16)
    g2r = h.alloc("g2r", [2, cap, K], torch.int64)
    rsv = h.alloc("rsv2", [cap, H], torch.bfloat16)
    src_h = torch.zeros(cap, H, dtype=torch.bfloat16)
    src_r = torch.zeros(cap, K, dtype=torch.int64)
    out = torch.zeros(cap, H, dtype=torch.bfloat16)
    p = DenseStepPlan(h, [g2h, g2r], [src_h, src_r], out, rsv, n_local, meta8, cap, 88)
    assert p.args.num_layers == 88 and p.args.dst_par_stride[0] == cap * H * 2 and p.args.ll_rows == 0
    with pytest.raises(ValueError):      # step_meta too short
        DenseStepPlan(h, [g2h], [src_h], out, rsv, n_local, torch.zeros(4, dtype=torch.int32), cap, 2)
    with pytest.raises(ValueError):      # gathered buffer without the parity dimension
        DenseStepPlan(h, [h.alloc("flat", [cap, H], torch.bfloat16)], [src_h], out, rsv, n_local, meta8, cap, 2)
    with pytest.raises(ValueError):      # pipeline groups need one block per SM
        DenseStepPlan(h, [g2h], [src_h], out, rsv, n_local, meta8, cap, 2, grid=296, groups=2)
    st_a = h.alloc("st_a", [agv_ll_stage_bytes(4, [H * 2, K * 8])], torch.uint8)
    st_r = h.alloc("st_r", [rsv_ll_stage_bytes(1, 4, cap, H * 2)], torch.uint8)
    with pytest.raises(ValueError):      # packet mode without its credit region
        DenseStepPlan(h, [g2h, g2r], [src_h, src_r], out, rsv, n_local, meta8, cap, 2, agv_ll_stage=st_a,
                      rsv_ll_stage=st_r, ll_rows=4)
    cr = h.alloc("cr", [step_credit_bytes(148)], torch.uint8)
    p = DenseStepPlan(h, [g2h, g2r], [src_h, src_r], out, rsv, n_local, meta8, cap, 2, agv_ll_stage=st_a,
                      rsv_ll_stage=st_r, ll_rows=4, credits=cr)
    assert p.args.ll_rows == 4 and p.args.credit_off == cr.offset
    # fp8 dispatch: uint8 rows + fp32 scales as a fourth tensor without a source
    q = h.alloc("q8", [2, cap, H], torch.uint8)
    sc = h.alloc("sc8", [2, cap, H // 128], torch.float32)
    g2p = h.alloc("g2p", [2, cap, K], torch.float32)
    src_p = torch.zeros(cap, K, dtype=torch.float32)
    p = DenseStepPlan(h, [q, g2r, g2p, sc], [src_h, src_r, src_p, None], out, rsv, n_local, meta8, cap, 2, fp8_hidden=H)
    assert p.args.fp8_hidden == H and p.args.row_bytes[0] == H and p.args.row_bytes[3] == H // 128 * 4 and p.args.src[3] is None
    with pytest.raises(ValueError):
        DenseStepPlan(h, [g2h, g2r, g2p, sc], [src_h, src_r, src_p, None], out, rsv, n_local, meta8, cap, 2, fp8_hidden=H)
    # all-to-all step
    assert a2a_meta_row_bytes(22) == 192 and a2a_meta_row_bytes(8) == 80
    for fp8 in (False, True):
        b = A2AStepBuffers(h, cap, H, K, fp8, prefix=f"t{int(fp8)}")
        assert b.recv_meta.tensor.shape == (2, 1, cap, a2a_meta_row_bytes(K))
        p = A2AStepPlan(h, b, src_h, src_r, src_p, out, n_local, meta8, 16, 88)
        assert p.args.x_par_stride == b.recv_x.nbytes // 2 and p.args.fp8 == int(fp8) and p.args.meta_row_bytes == 64
        assert (p.args.y_off == p.args.recv_x_off) == (not fp8)
        with pytest.raises(ValueError):
            A2AStepPlan(h, b, src_h[:4], src_r, src_p, out, n_local, meta8, 16, 88)
    st, tok, ids, wts = b.meta_fields(0, 0, 3)
    assert st.shape == (3,) and ids.shape == (3, K) and wts.dtype == torch.float32


def test_weight_tile_packing_round_trip():
    """The pre-packed weight layout: tile (row block, column block) is 16 KB of contiguous memory in the
    swizzled K-major shared-memory image; packing and unpacking are inverse, and chunk c of row r of a
    tile sits at chunk position c ^ (r % 8)."""
    from moe_comms_benchmarking_b200.ops.experts import ExpertWeights, pack_weight_tiles, unpack_weight_tiles
    w = torch.randn(3, 256, 192).to(torch.bfloat16)
    p = pack_weight_tiles(w)
    assert p.shape == (3, 2, 3, 128, 64) and p.is_contiguous()
    assert torch.equal(unpack_weight_tiles(p), w)
    for (e, rb, kb, r, c) in ((0, 0, 0, 0, 0), (1, 1, 2, 5, 3), (2, 0, 1, 127, 7), (2, 1, 0, 9, 6)):
        pos = c ^ (r % 8)
        assert torch.equal(p[e, rb, kb, r, pos * 8:pos * 8 + 8], w[e, rb * 128 + r, kb * 64 + c * 8:kb * 64 + c * 8 + 8])
    split = torch.arange(2 * 8 * 4, dtype=torch.float32).view(2, 8, 4)
    il = ExpertWeights.interleave(split)
    assert torch.equal(il[:, 0::2], split[:, :4]) and torch.equal(il[:, 1::2], split[:, 4:])
    with pytest.raises(ValueError):
        pack_weight_tiles(torch.zeros(1, 100, 64, dtype=torch.bfloat16))
