"""Symmetric heap: one allocation per rank, mapped into every peer and (with NVLS) bound
to an NVSwitch multicast object, plus a bump sub-allocator and a keyed registry.

Role of the reference's ``SymmetricMemoryManager`` / ``SymmetricMemoryBuffer``
(nvls/symmetric_memory.py:34-184).  Differences by design:

* ONE heap holds every buffer (the reference makes one symmetric allocation per tensor
  and always hands out offset 0, symmetric_memory.py:73-77), so a kernel needs one local
  base, one multicast base and one peer table, and names buffers by heap offset;
* the barrier flags live inside the heap with an explicit size
  (sites x blocks x 4 bytes), not in a library-sized signal pad;
* a heap also exists for a world of one and for CPU ranks (plain local memory), so the
  same dispatcher code runs at EP=1, in single-GPU emulation and under gloo.

PyTorch's CUDA symmetric memory is used as the host-side allocator for world > 1: it
creates the VMM allocation, exchanges handles and binds the multicast object; the kernels
only ever see raw addresses.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..ops import _ext

ALIGN = 256
FLAGS_BYTES = _ext.NUM_SITES * _ext.MAX_BLOCKS * 4
COUNTS_BYTES = 2 * _ext.MAX_RANKS * 4          # counts of the metadata kernel (two parities)
STEP_COUNTS_BYTES = 2 * _ext.MAX_RANKS * 4     # counts of the persistent dense step kernel (two parities)
A2A_COUNTS_BYTES = 2 * _ext.MAX_RANKS * 4      # counts of the persistent all-to-all step kernel
RESERVED_BYTES = ((FLAGS_BYTES + COUNTS_BYTES + STEP_COUNTS_BYTES + A2A_COUNTS_BYTES + ALIGN - 1) // ALIGN) * ALIGN


class DeviceStatusError(RuntimeError):
    """A kernel recorded an error in the status words (timeout, capacity, bounds, routing)."""

    def __init__(self, words):
        self.words = list(words)
        code, site, block, seen, wanted, rank = self.words[:6]
        name = _ext.ERR_NAMES.get(code, f"code{code}")
        super().__init__(f"device status: {name} at site {site} block {block} on rank {rank} "
                         f"(seen={seen}, wanted={wanted})")
        self.code = code


def _align(n: int, a: int = ALIGN) -> int:
    return (n + a - 1) // a * a


def required_bytes(specs) -> int:
    """Heap bytes needed for ``specs`` = iterable of (shape, dtype), including the reserved region."""
    total = RESERVED_BYTES
    for shape, dtype in specs:
        n = 1
        for s in shape:
            n *= int(s)
        total += _align(max(1, n * torch.empty((), dtype=dtype).element_size()))
    return total


@dataclass
class HeapTensor:
    tensor: torch.Tensor   # local view
    offset: int            # byte offset in the heap
    nbytes: int


class SymmetricHeap:
    """``SymmetricHeap(group, nbytes, device)`` is collective over ``group``."""

    def __init__(self, group, nbytes: int, device, transport: str = "auto", timeout_s: float = 2.0,
                 multicast: bool = True, allocator: str | None = None):
        """``multicast=False`` keeps the allocation out of any NVSwitch multicast object (peer
        mappings only).  Jobs in which a rank may leave while others keep running must use it: a
        rank that disappears while its memory is bound to a multicast object can raise NVLink
        faults on the surviving GPUs.  ``allocator``: ``"torch"`` (PyTorch's symmetric memory, the
        default) or ``"native"`` (this library's own allocator on the driver's virtual-memory API,
        ``parallel/native_heap.py``; one node); ``None`` reads ``MCB_HEAP_ALLOCATOR``."""
        self.group = group
        self.multicast = bool(multicast)
        self.device = torch.device(device)
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self.nbytes = _align(int(nbytes), 4096)
        self.timeout_s = timeout_s
        self.init_failure_reason = None
        self._handle = None
        self._cursor = RESERVED_BYTES
        self._registry: dict[str, HeapTensor] = {}
        self._reset_hooks = []
        self._site_grid: dict[int, int] = {}
        self.peer_ptrs = [0] * self.world
        self.mc_ptr = 0
        self._native = None
        allocator = allocator or os.environ.get("MCB_HEAP_ALLOCATOR", "torch")
        if allocator not in ("torch", "native"):
            raise ValueError(f"unknown heap allocator {allocator!r}")
        self.allocator = allocator
        on_gpu = self.device.type == "cuda"
        if self.world > 1 and on_gpu and allocator == "native":
            self._init_native()
        elif self.world > 1 and on_gpu:
            self._init_torch_symm()
        else:
            # World of one, or CPU ranks: an ordinary allocation is "symmetric" trivially.
            self.buffer = torch.zeros(self.nbytes, dtype=torch.uint8, device=self.device)
            self.peer_ptrs = [self.buffer.data_ptr()] if self.world == 1 else [0] * self.world
        if transport == "auto":
            transport = "multimem" if self.mc_ptr else "p2p"
        if transport == "multimem" and not self.mc_ptr:
            raise RuntimeError("multimem transport requested but no multicast address is available"
                               + (f" ({self.init_failure_reason})" if self.init_failure_reason else ""))
        if transport not in ("multimem", "p2p"):
            raise ValueError(f"unknown transport {transport!r}")
        self.transport = transport
        # Local (not symmetric) state: per-block epochs and the status words.
        self.epochs = torch.zeros(_ext.NUM_SITES * _ext.MAX_BLOCKS, dtype=torch.int32, device=self.device)
        self.status = torch.zeros(_ext.STATUS_WORDS, dtype=torch.int32, device=self.device)
        self._ctx = None

    # -- bring-up ---------------------------------------------------------------------------
    def _init_torch_symm(self):
        try:
            import torch.distributed._symmetric_memory as symm_mem
            try:
                symm_mem.enable_symm_mem_for_group(self.group.group_name)
            except Exception:
                pass  # newer versions need no opt-in
            # PyTorch binds a multicast object during the rendezvous unless this variable is set.
            prev = os.environ.get("TORCH_SYMM_MEM_DISABLE_MULTICAST")
            if not self.multicast:
                os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"
            try:
                self.buffer = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=self.device)
                self.buffer.zero_()
                self._handle = symm_mem.rendezvous(self.buffer, self.group.group_name)
            finally:
                if not self.multicast:
                    if prev is None:
                        os.environ.pop("TORCH_SYMM_MEM_DISABLE_MULTICAST", None)
                    else:
                        os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = prev
            self.peer_ptrs = [int(p) for p in self._handle.buffer_ptrs]
            self.mc_ptr = int(getattr(self._handle, "multicast_ptr", 0) or 0)
            if not self.multicast and self.mc_ptr:
                raise RuntimeError("a multicast address was bound although multicast=False was requested")
            if not self.mc_ptr:
                self.init_failure_reason = ("multicast disabled on request" if not self.multicast
                                            else "no NVLS multicast object for this group")
            torch.cuda.synchronize()
            dist.barrier(self.group)
        except Exception as e:  # surfaced by callers as a RuntimeError with the reason
            self.init_failure_reason = f"{type(e).__name__}: {e}"
            raise RuntimeError(f"symmetric heap bring-up failed: {self.init_failure_reason}") from e

    def _init_native(self):
        from .native_heap import NativeHeapBackend
        try:
            self._native = NativeHeapBackend(self.group, self.nbytes, self.device, multicast=self.multicast)
        except Exception as e:
            self.init_failure_reason = f"{type(e).__name__}: {e}"
            raise RuntimeError(f"symmetric heap bring-up failed: {self.init_failure_reason}") from e
        self.nbytes = self._native.nbytes
        self.buffer = self._native.buffer
        self.peer_ptrs = list(self._native.peer_ptrs)
        self.mc_ptr = self._native.mc_ptr
        if not self.mc_ptr:
            self.init_failure_reason = ("multicast disabled on request" if not self.multicast
                                        else "the devices of this group do not support multicast objects")

    # -- sub-allocation -----------------------------------------------------------------------
    def alloc(self, key: str, shape, dtype) -> HeapTensor:
        """Carve ``shape`` x ``dtype`` out of the heap under ``key``.  Every rank must call this
        in the same order with the same sizes so offsets agree.  Re-using a key returns the
        existing tensor if the size matches."""
        n = 1
        for s in shape:
            n *= int(s)
        esize = torch.empty((), dtype=dtype).element_size()
        nbytes = max(1, n * esize)
        if key in self._registry:
            ht = self._registry[key]
            if ht.nbytes != nbytes:
                raise ValueError(f"heap key {key!r} exists with {ht.nbytes} bytes, asked for {nbytes}")
            return ht
        off = self._cursor
        if off + nbytes > self.nbytes:
            raise MemoryError(f"symmetric heap exhausted: {key!r} needs {nbytes} bytes at offset {off}, "
                              f"heap has {self.nbytes}")
        self._cursor = _align(off + nbytes)
        view = self.buffer[off:off + n * esize].view(dtype).view(*shape)
        ht = HeapTensor(view, off, nbytes)
        self._registry[key] = ht
        return ht

    def get(self, key: str) -> HeapTensor:
        return self._registry[key]

    def bytes_used(self) -> int:
        return self._cursor

    @property
    def flags_off(self) -> int:
        return 0

    @property
    def counts_off(self) -> int:
        return FLAGS_BYTES

    @property
    def step_counts_off(self) -> int:
        return FLAGS_BYTES + COUNTS_BYTES

    @property
    def a2a_counts_off(self) -> int:
        return FLAGS_BYTES + COUNTS_BYTES + STEP_COUNTS_BYTES

    def peer_view(self, peer: int, ht: HeapTensor) -> torch.Tensor:
        """This rank's mapping of ``peer``'s copy of a heap tensor (debug / validation only)."""
        if peer == self.rank:
            return ht.tensor
        if self._native is not None:
            from .native_heap import _RawCudaBytes
            raw = _RawCudaBytes(self.peer_ptrs[peer] + ht.offset, ht.nbytes)
            t = torch.as_tensor(raw, device=self.device)
            t._mcb_keepalive = raw
            return t.view(ht.tensor.dtype).view(tuple(ht.tensor.shape))
        if self._handle is None:
            raise RuntimeError("no peer mappings on this heap")
        esize = ht.tensor.element_size()
        return self._handle.get_buffer(peer, tuple(ht.tensor.shape), ht.tensor.dtype, ht.offset // esize)

    # -- kernel context -------------------------------------------------------------------------
    def ctx(self) -> "_ext.McbCtx":
        if self._ctx is None:
            if self.world > _ext.MAX_RANKS:
                raise ValueError(f"world {self.world} exceeds MCB_MAX_RANKS {_ext.MAX_RANKS}")
            c = _ext.McbCtx()
            c.rank, c.world = self.rank, self.world
            c.transport = _ext.TRANSPORT_MULTIMEM if self.transport == "multimem" else _ext.TRANSPORT_P2P
            c.timeout_ns = int(self.timeout_s * 1e9)
            c.heap_local = self.buffer.data_ptr()
            c.heap_mc = self.mc_ptr
            c.flags_off = self.flags_off
            c.epochs = self.epochs.data_ptr()
            c.status = self.status.data_ptr()
            for p in range(self.world):
                c.heap_peer[p] = self.peer_ptrs[p]
            self._ctx = c
        return self._ctx

    def set_timeout(self, seconds: float):
        self.timeout_s = seconds
        self._ctx = None

    # -- health ------------------------------------------------------------------------------------
    def read_status(self) -> list[int]:
        return [int(v) & 0xFFFFFFFF for v in self.status.cpu().tolist()]

    def check_status(self):
        """Host-synchronising health check: raises ``DeviceStatusError`` if a kernel on this rank
        recorded an error.  The status words are cleared so the heap can be reused after
        ``reset_sync_state``."""
        words = self.read_status()
        if words[0] != 0:
            self.status.zero_()
            raise DeviceStatusError(words)

    def level_launch_counters(self, site: int, grid: int):
        """Kernels that number their launches with per-block counters (``next_launch_count``) need the
        same grid on every launch of a site.  Call this (on every rank, at the same point of the
        program, with nothing in flight on other streams) before the first launch with a new grid:
        it sets the site's whole counter row to its maximum, so blocks that did not exist under the
        old grid agree with the others.  A no-op while the grid stays the same."""
        if self._site_grid.get(site) == grid:
            return
        if site in self._site_grid:
            row = self.epochs[site * _ext.MAX_BLOCKS:(site + 1) * _ext.MAX_BLOCKS]
            row.fill_(int(row.max().item()))
        self._site_grid[site] = grid

    def register_reset_hook(self, fn):
        """``fn()`` runs on every rank inside ``reset_sync_state`` after the flags were cleared (for
        users of the heap that keep their own sequence words next to the flags)."""
        self._reset_hooks.append(fn)

    def reset_sync_state(self):
        """Collective: zero the flags and epochs on every rank (after an error, or between
        tests).  All kernels must have drained."""
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(self.group)
        self.buffer[:RESERVED_BYTES].zero_()
        # The launch counters of the low-latency paths keep counting: their value is the flag
        # carried by packets, and staging areas may still hold packets with earlier values.
        keep = {s: self.epochs[s * _ext.MAX_BLOCKS:(s + 1) * _ext.MAX_BLOCKS].clone() for s in _ext.LL_SITES}
        self.epochs.zero_()
        for s, v in keep.items():
            self.epochs[s * _ext.MAX_BLOCKS:(s + 1) * _ext.MAX_BLOCKS] = v
        self.status.zero_()
        for fn in self._reset_hooks:
            fn()
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(self.group)

    def destroy(self):
        """With the native allocator this is collective (the mappings of the peers go away)."""
        self._registry.clear()
        self._reset_hooks.clear()
        self._handle = None
        self.buffer = None
        if self._native is not None:
            self._native.close()
            self._native = None


class SymmetricHeapManager:
    """Keyed registry of heaps (role of SymmetricMemoryManager, symmetric_memory.py:133-184)."""

    _heaps: dict[str, SymmetricHeap] = {}

    @classmethod
    def get_heap(cls, key: str, group=None, nbytes: int = 512 << 20, device=None, **kw) -> SymmetricHeap:
        if key not in cls._heaps:
            if device is None:
                device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() \
                    else torch.device("cpu")
            cls._heaps[key] = SymmetricHeap(group, nbytes, device, **kw)
        return cls._heaps[key]

    @classmethod
    def destroy(cls, key: str | None = None):
        keys = [key] if key is not None else list(cls._heaps)
        for k in keys:
            h = cls._heaps.pop(k, None)
            if h is not None:
                h.destroy()

    @classmethod
    def is_initialized(cls, key: str) -> bool:
        return key in cls._heaps
