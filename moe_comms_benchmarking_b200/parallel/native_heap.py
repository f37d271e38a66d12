"""Host side of the native symmetric-heap allocator (csrc/symm_heap.cu).

The reference takes its symmetric buffer, peer pointers and multicast pointer from
torch.distributed._symmetric_memory (nvls/symmetric_memory.py:41-60).  ``NativeHeapBackend`` gets the same
three things from the driver's virtual-memory API through this library, without PyTorch's allocator: each
rank creates physical memory that can be shared as a file descriptor, the descriptors travel between the
ranks of the node over unix sockets (``SCM_RIGHTS``), every rank maps every peer's memory, and (optionally)
all of them bind their memory to one NVSwitch multicast object created by rank 0.

Selected with ``SymmetricHeap(..., allocator="native")`` or ``MCB_HEAP_ALLOCATOR=native``; PyTorch's
symmetric memory stays the default.  One node only (file descriptors do not cross machines).
"""
from __future__ import annotations

import array
import ctypes as C
import os
import socket
import struct

import torch
import torch.distributed as dist

from ..ops import _ext

_ERRLEN = 256


class NativeHeapError(RuntimeError):
    pass


def _check(rc: int, err) -> None:
    if rc != 0:
        raise NativeHeapError(f"native heap: {err.value.decode(errors='replace')} [{rc}]")


class _RawCudaBytes:
    """Lets ``torch.as_tensor`` wrap a raw device address (the mapping is owned by the heap object)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def _send_fds(sock: socket.socket, payload: bytes, fds: list[int]) -> None:
    sock.sendmsg([payload], [(socket.SOL_SOCKET, socket.SCM_RIGHTS, array.array("i", fds))])


def _recv_fds(sock: socket.socket, nbytes: int, maxfds: int) -> tuple[bytes, list[int]]:
    fds = array.array("i")
    msg, anc, _flags, _addr = sock.recvmsg(nbytes, socket.CMSG_LEN(maxfds * fds.itemsize))
    for level, ctype, data in anc:
        if level == socket.SOL_SOCKET and ctype == socket.SCM_RIGHTS:
            fds.frombytes(data[:len(data) - (len(data) % fds.itemsize)])
    return msg, list(fds)


def exchange_fds(group, rank: int, world: int, own_fds: list[int], tag: str) -> dict[int, list[int]]:
    """Every rank sends ``own_fds`` to every other rank of the node; returns {peer: its descriptors as
    received here}.  Each rank listens on an abstract unix socket named after ``tag`` and its rank; all
    connect and send first (the connections wait in the listeners' backlog), then all accept."""
    name = lambda r: f"\0mcb-heap-{tag}-{r}"          # abstract namespace: nothing to unlink
    srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    srv.bind(name(rank))
    srv.listen(world)
    srv.settimeout(60.0)
    dist.barrier(group)                                # every listener exists
    outs = []
    try:
        for p in range(world):
            if p == rank:
                continue
            c = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            c.settimeout(60.0)
            c.connect(name(p))
            _send_fds(c, struct.pack("ii", rank, len(own_fds)), own_fds)
            outs.append(c)
        got: dict[int, list[int]] = {}
        for _ in range(world - 1):
            conn, _ = srv.accept()
            conn.settimeout(60.0)
            msg, fds = _recv_fds(conn, 8, 4)
            src, n = struct.unpack("ii", msg)
            if len(fds) != n:
                raise NativeHeapError(f"rank {src} announced {n} descriptors, {len(fds)} arrived")
            got[src] = fds
            conn.close()
    finally:
        dist.barrier(group)                            # every message has been received: senders may close
        for c in outs:
            c.close()
        srv.close()
    return got


class NativeHeapBackend:
    """Collective over ``group`` (one node).  Attributes after construction: ``buffer`` (uint8 tensor over
    the local mapping), ``peer_ptrs`` (this rank's address of every rank's memory), ``mc_ptr`` (multicast
    address or 0), ``nbytes`` (size rounded up to the driver's granularity)."""

    def __init__(self, group, nbytes: int, device: torch.device, multicast: bool = True):
        lib = _ext.require()
        if not lib.mcb_nheap_available():
            raise NativeHeapError("the CUDA driver library (libcuda.so.1) or one of its virtual-memory entry points is missing")
        self.group, self.device = group, device
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self._lib = lib
        self._heap = C.c_void_p()
        self._closed = False
        err = C.create_string_buffer(_ERRLEN)
        torch.cuda.set_device(device)
        torch.zeros(1, device=device)                  # the primary context exists and is current
        index = device.index if device.index is not None else torch.cuda.current_device()
        want_mc = bool(multicast) and self.world > 1
        if want_mc:
            sup = torch.tensor([int(lib.mcb_nheap_multicast_supported(index) == 1)], device=device)
            dist.all_reduce(sup, op=dist.ReduceOp.MIN, group=group)
            want_mc = bool(int(sup.item()))
        size, ptr, fd = C.c_ulonglong(), C.c_ulonglong(), C.c_int(-1)
        _check(lib.mcb_nheap_create(index, C.c_ulonglong(int(nbytes)), self.world, int(want_mc), C.byref(self._heap),
                                    C.byref(size), C.byref(ptr), C.byref(fd), err, _ERRLEN), err)
        self.nbytes = int(size.value)
        own = [fd.value]
        mc_fd = C.c_int(-1)
        if want_mc and self.rank == 0:
            _check(lib.mcb_nheap_mc_create(self._heap, self.world, C.byref(mc_fd), err, _ERRLEN), err)
            own.append(mc_fd.value)
        # one tag for the whole job: rank 0's process id and a counter of heaps built so far
        box = [f"{os.getpid()}-{NativeHeapBackend._serial}"] if self.rank == 0 else [None]
        dist.broadcast_object_list(box, src=0, group=group)
        NativeHeapBackend._serial += 1
        received = exchange_fds(group, self.rank, self.world, own, box[0])
        self.peer_ptrs = [0] * self.world
        self.peer_ptrs[self.rank] = int(ptr.value)
        try:
            for p, fds in sorted(received.items()):
                pp = C.c_ulonglong()
                _check(lib.mcb_nheap_map_peer(self._heap, fds[0], C.byref(pp), err, _ERRLEN), err)
                self.peer_ptrs[p] = int(pp.value)
                if want_mc and p == 0 and self.rank != 0:
                    if len(fds) < 2:
                        raise NativeHeapError("rank 0 sent no multicast descriptor")
                    _check(lib.mcb_nheap_mc_import(self._heap, fds[1], err, _ERRLEN), err)
        finally:
            for fds in received.values():
                for f in fds:
                    os.close(f)
            for f in own:
                os.close(f)
        self.mc_ptr = 0
        if want_mc:
            _check(lib.mcb_nheap_mc_add_device(self._heap, err, _ERRLEN), err)
            dist.barrier(group)                        # every device is part of the object before anyone binds
            mc = C.c_ulonglong()
            _check(lib.mcb_nheap_mc_bind(self._heap, C.byref(mc), err, _ERRLEN), err)
            self.mc_ptr = int(mc.value)
        self._raw = _RawCudaBytes(int(ptr.value), self.nbytes)
        self.buffer = torch.as_tensor(self._raw, device=device)
        self.buffer.zero_()
        torch.cuda.synchronize()
        dist.barrier(group)

    _serial = 0

    def close(self):
        """Collective: nobody may touch a peer's memory or the multicast address afterwards."""
        if self._closed:
            return
        self._closed = True
        torch.cuda.synchronize()
        dist.barrier(self.group)
        self.buffer = None
        self._lib.mcb_nheap_destroy(self._heap)
        self._heap = C.c_void_p()
