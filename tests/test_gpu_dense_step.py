"""The persistent decode-step kernel (count exchange + every layer in one launch), emulated as W
ranks inside one cooperative launch on ONE GPU, against the CPU oracle; plus its race test: the
self-checking build with per-rank delays chosen on the host, alternating packet and barrier steps."""
import pytest
import torch

from moe_comms_benchmarking_b200.ops import _ext, oracle
from moe_comms_benchmarking_b200.ops.dense import agv_ll_stage_bytes, rsv_ll_stage_bytes
from moe_comms_benchmarking_b200.parallel.emulation import EmuWorld
from moe_comms_benchmarking_b200.parallel.symm_heap import DeviceStatusError

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _scalars(vals):
    return [torch.tensor([v], dtype=torch.int32, device=DEV) for v in vals]


class _Rig:
    """Buffers of an emulated dense dispatcher: [2, cap*W, cols] gathered tensors per rank."""

    def __init__(self, W, cap, H, K, LL, dtype=torch.bfloat16):
        self.W, self.cap, self.H, self.K, self.LL = W, cap, H, K, LL
        self.w = EmuWorld(W, 16 << 20, DEV)
        self.dst_h = self.w.alloc([2, cap * W, H], torch.bfloat16)
        self.dst_r = self.w.alloc([2, cap * W, K], torch.int64)
        self.dst_p = self.w.alloc([2, cap * W, K], torch.float32)
        self.rsv = self.w.alloc([cap * W, H], dtype)
        self.st_a = self.w.alloc([max(16, agv_ll_stage_bytes(LL, [H * 2, K * 8, K * 4]))], torch.uint8)
        self.st_r = self.w.alloc([max(16, rsv_ll_stage_bytes(W, LL, cap, H * 2))], torch.uint8)
        self.metas = [torch.zeros(8, dtype=torch.int32, device=DEV) for _ in range(W)]
        self.outs = [torch.zeros(cap, H, dtype=dtype, device=DEV) for _ in range(W)]
        self.g = torch.Generator(device=DEV).manual_seed(77)
        self.dtype = dtype

    def new_inputs(self):
        W, cap, H, K, g = self.W, self.cap, self.H, self.K, self.g
        self.src_h = [torch.randn(cap, H, device=DEV, generator=g).to(torch.bfloat16) for _ in range(W)]
        self.src_r = [torch.randint(0, 512, (cap, K), device=DEV, generator=g) for _ in range(W)]
        self.src_p = [torch.rand(cap, K, device=DEV, generator=g) for _ in range(W)]
        for r in range(W):
            self.rsv[r].tensor.copy_(torch.randn(cap * W, H, device=DEV, generator=g).to(self.dtype))

    def step(self, counts, layers, grid, threads, groups=1, **kw):
        self.w.dense_step([self.dst_h, self.dst_r, self.dst_p], [self.src_h, self.src_r, self.src_p], self.outs,
                          self.rsv, _scalars(counts), self.metas, self.cap, layers, grid=grid, threads=threads,
                          agv_ll_stage=self.st_a, rsv_ll_stage=self.st_r, ll_rows=self.LL, groups=groups,
                          group_min_bytes=0, **kw)

    def check(self, counts, expect_mode=None, tol=2e-2):
        W = self.W
        valid = sum(counts)
        want_meta = oracle.metadata(counts)
        full = [oracle.all_gather_v([s[r][:counts[r]] for r in range(W)]) for s in (self.src_h, self.src_r, self.src_p)]
        want = oracle.reduce_scatter_v([self.rsv[r].tensor[:valid].cpu() for r in range(W)], counts)
        for r in range(W):
            m = self.metas[r].tolist()
            assert m[:3] == want_meta[r]
            if expect_mode is not None:
                assert m[6] == expect_mode
            par = m[5]
            assert torch.equal(self.dst_h[r].tensor[par, :valid], full[0])
            assert torch.equal(self.dst_r[r].tensor[par, :valid], full[1])
            assert torch.equal(self.dst_p[r].tensor[par, :valid], full[2])
            assert torch.allclose(self.outs[r][:counts[r]].float().cpu(), want[r], rtol=tol, atol=tol)


@pytest.mark.parametrize("grid,threads,groups", [(1, 128, 1), (8, 256, 1), (8, 256, 2), (12, 128, 3)])
def test_step_kernel_barrier_and_packet_modes(lib, grid, threads, groups):
    """Steps of 1-3 layers on the same buffers, switching between packet mode (<= 8 rows in total)
    and barrier mode, with idle ranks and an empty step; every step against the oracle."""
    rig = _Rig(W=4, cap=16, H=256, K=22, LL=8)
    plan = [([5, 0, 16, 3], 3, 0), ([1, 2, 3, 2], 2, 1), ([1, 0, 0, 0], 3, 1), ([16, 16, 16, 16], 1, 0),
            ([0, 0, 0, 0], 2, None), ([0, 8, 0, 0], 5, 1), ([4, 4, 4, 4], 2, 0), ([2, 2, 2, 2], 4, 1)]
    for counts, layers, mode in plan:
        rig.new_inputs()
        rig.step(counts, layers, grid, threads, groups)
        rig.check(counts, expect_mode=mode)
        if mode == 0 and groups > 1 and grid >= 2 * groups:
            assert rig.metas[0][7].item() == groups
    rig.w.check_status()


def test_step_kernel_grid_may_change_between_steps(lib):
    """The sequence words live outside the per-block counters, so a step may use another grid size
    than the one before (packet flags and barrier targets stay in agreement)."""
    rig = _Rig(W=2, cap=32, H=256, K=22, LL=8)
    for counts, layers, grid in (([3, 2], 3, 4), ([3, 2], 3, 16), ([20, 32], 2, 2), ([20, 32], 2, 24), ([4, 4], 3, 8)):
        rig.new_inputs()
        rig.step(counts, layers, grid, 256)
        rig.check(counts)
    rig.w.check_status()


def test_step_kernel_fp32_combine(lib):
    rig = _Rig(W=2, cap=8, H=128, K=4, LL=0, dtype=torch.float32)
    rig.new_inputs()
    rig.step([3, 8], 2, 4, 128)
    rig.check([3, 8], expect_mode=0, tol=1e-5)
    rig.w.check_status()


@pytest.mark.parametrize("grid,threads", [(2, 128), (8, 256)])
def test_step_kernel_fp8_dispatch(lib, grid, threads):
    """1 x 128 block-scaled e4m3 dispatch inside the step kernel, in barrier mode and in packet mode:
    scales == amax / 448, values within e4m3 rounding of the inputs (against the CPU oracle's
    quantiser), routing / probs bit-exact, combine unaffected."""
    W, cap, H, K, LL = 4, 16, 512, 6, 8
    w = EmuWorld(W, 16 << 20, DEV)
    dst_q = w.alloc([2, cap * W, H], torch.uint8)
    dst_r = w.alloc([2, cap * W, K], torch.int64)
    dst_p = w.alloc([2, cap * W, K], torch.float32)
    dst_s = w.alloc([2, cap * W, H // 128], torch.float32)
    rsv = w.alloc([cap * W, H], torch.bfloat16)
    st_a = w.alloc([agv_ll_stage_bytes(LL, [H, K * 8, K * 4, H // 128 * 4])], torch.uint8)
    st_r = w.alloc([rsv_ll_stage_bytes(W, LL, cap, H * 2)], torch.uint8)
    metas = [torch.zeros(8, dtype=torch.int32, device=DEV) for _ in range(W)]
    outs = [torch.zeros(cap, H, dtype=torch.bfloat16, device=DEV) for _ in range(W)]
    g = torch.Generator(device=DEV).manual_seed(5)
    for counts, layers, mode in (([5, 0, 16, 3], 2, 0), ([1, 2, 3, 2], 3, 1), ([16, 16, 16, 16], 1, 0), ([0, 1, 0, 0], 2, 1)):
        src_h = [(torch.randn(cap, H, device=DEV, generator=g) * (1 + r)).to(torch.bfloat16) for r in range(W)]
        src_h[1][0, :128] = 0                      # an all-zero block
        src_r = [torch.randint(0, 512, (cap, K), device=DEV, generator=g) for _ in range(W)]
        src_p = [torch.rand(cap, K, device=DEV, generator=g) for _ in range(W)]
        for r in range(W):
            rsv[r].tensor.copy_(torch.randn(cap * W, H, device=DEV, generator=g).to(torch.bfloat16))
        w.dense_step([dst_q, dst_r, dst_p, dst_s], [src_h, src_r, src_p, None], outs, rsv, _scalars(counts), metas, cap,
                     layers, grid=grid, threads=threads, agv_ll_stage=st_a, rsv_ll_stage=st_r, ll_rows=LL, fp8_hidden=H)
        valid = sum(counts)
        full_h = oracle.all_gather_v([src_h[r][:counts[r]] for r in range(W)]).float().cpu()
        full_r = oracle.all_gather_v([src_r[r][:counts[r]] for r in range(W)])
        full_p = oracle.all_gather_v([src_p[r][:counts[r]] for r in range(W)])
        q_ref, s_ref = oracle.quant_e4m3_1x128(full_h)
        want = oracle.reduce_scatter_v([rsv[r].tensor[:valid].cpu() for r in range(W)], counts)
        for r in range(W):
            m = metas[r].tolist()
            assert m[6] == mode
            par = m[5]
            sc = dst_s[r].tensor[par, :valid].cpu()
            q = dst_q[r].tensor[par, :valid].cpu().view(torch.float8_e4m3fn)
            assert torch.allclose(sc, s_ref, rtol=1e-6, atol=0)
            back = oracle.dequant_e4m3_1x128(q, sc)
            assert ((back - full_h).abs() <= 0.0625 * full_h.abs() + 2e-3 * sc.repeat_interleave(128, dim=1)).all()
            assert (q.float() == q_ref.float()).float().mean() > 0.999
            assert torch.equal(dst_r[r].tensor[par, :valid], full_r) and torch.equal(dst_p[r].tensor[par, :valid], full_p)
            assert torch.allclose(outs[r][:counts[r]].float().cpu(), want[r], rtol=2e-2, atol=2e-2)
    w.check_status()


def test_step_kernel_bounded_wait_with_a_phantom_rank(lib):
    """A world that counts a rank which never runs: the count exchange cannot complete, the
    bounded wait runs out, the status words say so and the GPU context stays usable."""
    W, cap, H, K = 2, 4, 128, 4
    w = EmuWorld(W, 1 << 20, DEV, timeout_s=0.2, phantom_ranks=1)
    T = W + 1
    dst = [w.alloc([2, cap * T, c], dt) for c, dt in ((H, torch.bfloat16), (K, torch.int64), (K, torch.float32))]
    rsv = w.alloc([cap * T, H], torch.bfloat16)
    srcs = [[torch.zeros(cap, c, dtype=dt, device=DEV) for _ in range(W)]
            for c, dt in ((H, torch.bfloat16), (K, torch.int64), (K, torch.float32))]
    outs = [torch.zeros(cap, H, dtype=torch.bfloat16, device=DEV) for _ in range(W)]
    metas = [torch.zeros(8, dtype=torch.int32, device=DEV) for _ in range(W)]
    w.dense_step(dst, srcs, outs, rsv, _scalars([1, 1]), metas, cap, 2, grid=2, threads=128)
    with pytest.raises(DeviceStatusError) as e:
        w.check_status()
    assert e.value.code == 1 and e.value.words[1] == _ext.SITE_STEP_META
    assert torch.ones(4, device=DEV).sum().item() == 4.0     # the context still works


@pytest.mark.parametrize("groups", [1, 2])
def test_step_kernel_race_check_with_delays(lib, groups):
    """Write-after-read stress: >= 200 layers in steps that alternate between packet mode and
    barrier mode, self-checking payload (a hash of the layer number and the position, verified by
    every receiver right after its barrier or poll), and a different rank slowed down in every step
    by a bounded sleep per layer.  A push that overtakes a reader, or a stale packet, is a mismatch."""
    W, cap, LL = 4, 16, 8
    rig = _Rig(W, cap, H=256, K=22, LL=LL)
    rig.new_inputs()
    errs = [torch.zeros(1, dtype=torch.int32, device=DEV) for _ in range(W)]
    layers_done = 0
    step = 0
    while layers_done < 220:
        packet = step % 2 == 0
        counts = [[2, 1, 0, 3], [1, 1, 1, 1], [0, 0, 5, 0]][step % 3] if packet else \
                 [[16, 9, 0, 12], [7, 16, 16, 1]][(step // 2) % 2]
        layers = 5 + step % 4
        delays = [0] * W
        delays[step % W] = 20000 + 3000 * (step % 5)
        delays[(step + 2) % W] = 7000
        rig.step(counts, layers, 8, 256, groups, check_errors=errs, delays_ns=delays, delay_every=1 + step % 3)
        for r in range(W):
            assert rig.metas[r][6].item() == (1 if packet else 0)
        layers_done += layers
        step += 1
    rig.w.check_status()
    assert [int(e.item()) for e in errs] == [0] * W
    # the combine of the last step is the real one (only the gathered payload is synthetic)
    want = oracle.reduce_scatter_v([rig.rsv[r].tensor[:sum(counts)].cpu() for r in range(W)], counts)
    for r in range(W):
        assert torch.allclose(rig.outs[r][:counts[r]].float().cpu(), want[r], rtol=2e-2, atol=2e-2)


def test_step_kernel_check_payload_depends_on_the_layer(lib):
    """The self-checking payload is a function of the layer number: two consecutive one-layer steps
    leave different words in the two parities of the gathered buffer, identical on all ranks."""
    rig = _Rig(W=2, cap=8, H=128, K=4, LL=0)
    rig.new_inputs()
    errs = [torch.zeros(1, dtype=torch.int32, device=DEV) for _ in range(2)]
    rig.step([4, 4], 1, 2, 128, check_errors=errs)
    par = rig.metas[1][5].item()
    first = rig.dst_h[1].tensor[par, :8].view(torch.int16).clone()      # raw words (the hash may spell NaNs)
    assert torch.equal(first, rig.dst_h[0].tensor[par, :8].view(torch.int16)) and first.count_nonzero().item() > 0
    rig.step([4, 4], 1, 2, 128, check_errors=errs)
    par2 = rig.metas[1][5].item()
    assert par2 != par and not torch.equal(rig.dst_h[1].tensor[par2, :8].view(torch.int16), first)
    assert [int(e.item()) for e in errs] == [0, 0]
    rig.w.check_status()
