"""The allocation-free dispatch entry point, called through its exported C symbol.

Some users of the library launch from places where they cannot allocate GPU memory (their
memory comes from a pool filled at start-up, or they sit on a latency path where an allocation
could stall the device).  For them ``mcb_a2a_dispatch_noalloc`` keeps the kernel's scratch
counters in an array inside the library.  This test runs the ordinary entry point and the
allocation-free one on the same tokens and requires the same received rows, row counts,
routing rows and slot map; the allocation-free call is made twice in a row because both calls
share the one scratch array.  Collected last on purpose, so that a run that stops at the first
failure has already exercised everything else.
"""
import ctypes as C
import gc

import pytest
import torch

pytestmark = pytest.mark.gpu


def _received(bufs, n):
    """Rows received from source 0 in source-token order (slots are handed out by an atomic
    counter, so their order differs from launch to launch)."""
    c = int(bufs.recv_count.tensor[0])
    order = torch.argsort(bufs.recv_src.tensor[0, :c].long())
    return (c, bufs.recv_src.tensor[0, :c][order].clone(), bufs.recv_x.tensor[0, :c][order].clone(),
            bufs.recv_idx.tensor[0, :c][order].clone(), bufs.recv_w.tensor[0, :c][order].clone())


def test_no_alloc_dispatch_matches_the_ordinary_entry_point(world1, lib):
    from moe_comms_benchmarking_b200.config import Config
    from moe_comms_benchmarking_b200.ops import _ext
    from moe_comms_benchmarking_b200.parallel.a2a import A2ADispatcher
    from moe_comms_benchmarking_b200.utils.inputs import make_inputs

    cfg = Config(ep_size=1, rank=0, local_rank=0, per_rank_cap=96)
    d = A2ADispatcher(cfg, world1)
    d.build()
    n = 77
    h, i, w = make_inputs(cfg, n, "cuda:0")
    d.setup_batch(h, i, w)

    d.dispatch()                                   # the existing entry point
    torch.cuda.synchronize()
    want = _received(d.bufs, n)
    want_slots = d.bufs.slot_map[:n].clone()
    assert want[0] == n and torch.equal(want[2], h)

    lib.mcb_a2a_dispatch_noalloc.restype = C.c_int
    lib.mcb_noalloc_last_error.restype = C.c_char_p
    assert lib.mcb_noalloc_scratch_bytes() == 4 * (lib.mcb_noalloc_max_ranks() + 1)
    args = d.dispatch_plan.args
    poisoned = torch.full((_ext.MAX_RANKS + 1,), 12345, dtype=torch.int32, device="cuda:0")
    for call in range(2):
        # wipe what the previous call produced, and point the caller-side scratch field at
        # garbage: the entry point must not use it
        d.bufs.recv_x.tensor.zero_()
        d.bufs.recv_idx.tensor.zero_()
        d.bufs.recv_w.tensor.zero_()
        d.bufs.recv_src.tensor.fill_(-1)
        d.bufs.recv_count.tensor.fill_(-1)
        d.bufs.slot_map.fill_(-7)
        mine = _ext.McbA2ADispatchArgs.from_buffer_copy(args)
        mine.send_count = poisoned.data_ptr()
        # Objects left over from earlier tests must not be collected (and their GPU memory
        # freed) inside the window in which the allocator's counter is compared.
        gc.collect()
        gc.disable()
        try:
            before = torch.cuda.memory_allocated()
            free_before = torch.cuda.mem_get_info()[0]
            rc = lib.mcb_a2a_dispatch_noalloc(C.byref(d.heap.ctx()), C.byref(mine), d.num_sms, d.threads,
                                              _ext.stream_handle())
            assert rc == 0, lib.mcb_noalloc_last_error().decode()
            torch.cuda.synchronize()
            free_after = torch.cuda.mem_get_info()[0]
            assert torch.cuda.memory_allocated() == before
            # PyTorch's counter above cannot see an allocation made inside the library; the driver's
            # free-memory figure can (a cudaMalloc takes at least one 2 MiB block from it).  The first
            # call on a device may load the kernel image, so the figure is compared on the second.
            if call == 1:
                assert free_after >= free_before, f"device memory shrank by {free_before - free_after} bytes"
        finally:
            gc.enable()
        got = _received(d.bufs, n)
        assert got[0] == want[0], f"call {call}: row count"
        for g, x in zip(got[1:], want[1:]):
            assert torch.equal(g, x), f"call {call}"
        # at world 1 every token takes one slot on rank 0: the slot map is a permutation of 0..n-1
        assert sorted(d.bufs.slot_map[:n, 0].tolist()) == sorted(want_slots[:, 0].tolist()) == list(range(n))
        assert torch.all(poisoned == 12345)
    d.check_health()

    # a world larger than the built-in scratch holds is refused with a reason, nothing is launched
    big = _ext.McbCtx.from_buffer_copy(d.heap.ctx())
    big.world = _ext.MAX_RANKS + 1
    rc = lib.mcb_a2a_dispatch_noalloc(C.byref(big), C.byref(mine), d.num_sms, d.threads, _ext.stream_handle())
    assert rc != 0 and "world size" in lib.mcb_noalloc_last_error().decode()
    torch.cuda.synchronize()
    d.destroy()
