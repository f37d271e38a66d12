"""Host side of the native symmetric-heap allocator, on CPU ranks: the file descriptors that carry the
memory handles travel over unix sockets between gloo ranks (here: pipe ends, checked by writing through
them), and the library reports a missing GPU driver instead of failing to load."""
import os

import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import free_port


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    from moe_comms_benchmarking_b200.parallel.dist import init_distributed
    from moe_comms_benchmarking_b200.parallel.native_heap import exchange_fds
    group, r, w, _ = init_distributed(backend="gloo")
    rd, wr = os.pipe()
    own = [wr] if r else [wr, os.dup(wr)]              # rank 0 sends two descriptors, like memory + multicast object
    got = exchange_fds(group, r, w, own, f"test-{port}")
    ok = sorted(got) == [p for p in range(w) if p != r]
    ok = ok and all(len(got[p]) == (2 if p == 0 else 1) for p in got)
    for p, fds in got.items():                         # write through the received write ends
        os.write(fds[0], bytes([r]))
    dist.barrier(group)
    seen = sorted(os.read(rd, 64))                     # every other rank wrote its number into my pipe
    ok = ok and seen == [p for p in range(w) if p != r]
    q.put((r, ok))
    dist.barrier(group)
    dist.destroy_process_group()


def test_descriptor_exchange_between_three_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, 3, port, q)) for r in range(3)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok in res), res


def test_library_reports_a_missing_driver_instead_of_failing():
    import ctypes as C
    from moe_comms_benchmarking_b200.ops import _ext
    lib = _ext.load()
    avail = lib.mcb_nheap_available()
    assert avail in (0, 1)
    if not avail:                                      # no GPU driver on this machine: creation is refused with a reason
        heap, size, ptr, fd = C.c_void_p(), C.c_ulonglong(), C.c_ulonglong(), C.c_int(-1)
        err = C.create_string_buffer(256)
        rc = lib.mcb_nheap_create(0, C.c_ulonglong(1 << 20), 1, 0, C.byref(heap), C.byref(size), C.byref(ptr),
                                  C.byref(fd), err, 256)
        assert rc != 0 and b"libcuda" in err.value and not heap.value
