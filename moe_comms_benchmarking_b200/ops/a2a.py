"""All-to-all-V dispatch/combine plans (peer stores / peer loads, optional e4m3 dispatch).

Plays the role of the ``deep_ep.ElasticBuffer.dispatch`` / ``.combine`` calls the reference
wraps (bench_deepep.py:36-94): one copy per distinct destination rank, device-side count
exchange, combine tied to the routing of the dispatch before it (here through ``slot_map``).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _ext
from .dense import DEFAULT_GRID, DEFAULT_THREADS, _check_grid, _check_heap_tensor
from ..parallel.symm_heap import SymmetricHeap


class A2ABuffers:
    """Heap and local buffers of one all-to-all dispatcher.  Receive layout on every rank:
    ``[source rank][cap][...]``; ``recv_count[s]`` rows of source ``s`` are valid."""

    def __init__(self, heap: SymmetricHeap, cap: int, hidden: int, topk: int, fp8: bool, prefix: str = "a2a"):
        w = heap.world
        dev = heap.device
        self.cap, self.hidden, self.topk, self.fp8 = cap, hidden, topk, fp8
        if hidden % 8 or (fp8 and hidden % 128):
            raise ValueError("hidden must be a multiple of 8 (128 with fp8 dispatch)")
        if fp8:
            self.recv_x = heap.alloc(f"{prefix}_recv_x8", [w, cap, hidden], torch.uint8)
            self.recv_scale = heap.alloc(f"{prefix}_recv_scale", [w, cap, hidden // 128], torch.float32)
            self.y = heap.alloc(f"{prefix}_y", [w, cap, hidden], torch.bfloat16)
        else:
            self.recv_x = heap.alloc(f"{prefix}_recv_x", [w, cap, hidden], torch.bfloat16)
            self.recv_scale = None
            self.y = self.recv_x       # identity expert: combine reads the received rows
        self.recv_idx = heap.alloc(f"{prefix}_recv_idx", [w, cap, topk], torch.int64)
        self.recv_w = heap.alloc(f"{prefix}_recv_w", [w, cap, topk], torch.float32)
        self.recv_src = heap.alloc(f"{prefix}_recv_src", [w, cap], torch.int32)
        self.recv_count = heap.alloc(f"{prefix}_recv_count", [_ext.MAX_RANKS], torch.int32)
        self.slot_map = torch.full((cap, w), -1, dtype=torch.int32, device=dev)
        self.send_count = torch.zeros(_ext.MAX_RANKS + 1, dtype=torch.int32, device=dev)

    @staticmethod
    def specs(world: int, cap: int, hidden: int, topk: int, fp8: bool):
        s = [([world, cap, topk], torch.int64), ([world, cap, topk], torch.float32),
             ([world, cap], torch.int32), ([_ext.MAX_RANKS], torch.int32)]
        if fp8:
            s += [([world, cap, hidden], torch.uint8), ([world, cap, hidden // 128], torch.float32),
                  ([world, cap, hidden], torch.bfloat16)]
        else:
            s += [([world, cap, hidden], torch.bfloat16)]
        return s


class A2ADispatchPlan:
    def __init__(self, heap: SymmetricHeap, bufs: A2ABuffers, x, topk_idx, topk_w, n_local, num_experts: int,
                 grid: int = DEFAULT_GRID, threads: int = DEFAULT_THREADS):
        _check_grid(grid, threads)
        if x.dtype != torch.bfloat16 or x.dim() != 2 or x.shape[1] != bufs.hidden or not x.is_contiguous():
            raise ValueError("x must be contiguous bf16 [rows, hidden]")
        if topk_idx.dtype != torch.int64 or topk_idx.shape[1] != bufs.topk or not topk_idx.is_contiguous():
            raise ValueError("topk_idx must be contiguous int64 [rows, topk]")
        if topk_w is not None and (topk_w.dtype != torch.float32 or not topk_w.is_contiguous()):
            raise ValueError("topk_w must be contiguous fp32 [rows, topk]")
        if x.shape[0] < bufs.cap or topk_idx.shape[0] < bufs.cap:
            raise ValueError("input buffers must hold `cap` rows")
        if num_experts % heap.world:
            raise ValueError("num_experts must be divisible by the world size")
        for name in ("recv_x", "recv_idx", "recv_w", "recv_src", "recv_count"):
            _check_heap_tensor(heap, getattr(bufs, name), name)
        self.heap, self.bufs, self.grid, self.threads = heap, bufs, grid, threads
        self._keep = (x, topk_idx, topk_w, n_local)
        a = _ext.McbA2ADispatchArgs()
        a.x, a.topk_idx, a.topk_w = x.data_ptr(), topk_idx.data_ptr(), _ext.ptr(topk_w)
        a.recv_x_off = bufs.recv_x.offset
        a.recv_scale_off = bufs.recv_scale.offset if bufs.recv_scale is not None else 0
        a.recv_idx_off, a.recv_w_off = bufs.recv_idx.offset, bufs.recv_w.offset
        a.recv_src_off, a.recv_count_off = bufs.recv_src.offset, bufs.recv_count.offset
        a.slot_map, a.send_count = bufs.slot_map.data_ptr(), bufs.send_count.data_ptr()
        a.n_local = n_local.data_ptr()
        a.hidden, a.topk, a.num_experts, a.cap = bufs.hidden, bufs.topk, int(num_experts), bufs.cap
        a.fp8 = 1 if bufs.fp8 else 0
        self.args = a

    def launch(self, pdl: bool = False, stream=None):
        lib = _ext.require()
        _ext.check(lib.mcb_launch_a2a_dispatch(C.byref(self.heap.ctx()), C.byref(self.args), self.grid,
                                               self.threads, int(pdl), _ext.stream_handle(stream)),
                   "a2a_dispatch")


class A2ACombinePlan:
    def __init__(self, heap: SymmetricHeap, bufs: A2ABuffers, out, n_local,
                 grid: int = DEFAULT_GRID, threads: int = DEFAULT_THREADS):
        _check_grid(grid, threads)
        if out.dtype != torch.bfloat16 or out.shape[1] != bufs.hidden or out.shape[0] < bufs.cap:
            raise ValueError("out must be bf16 [cap, hidden]")
        _check_heap_tensor(heap, bufs.y, "y")
        self.heap, self.bufs, self.grid, self.threads = heap, bufs, grid, threads
        self._keep = (out, n_local)
        a = _ext.McbA2ACombineArgs()
        a.out, a.y_off = out.data_ptr(), bufs.y.offset
        a.slot_map, a.n_local = bufs.slot_map.data_ptr(), n_local.data_ptr()
        a.hidden, a.cap = bufs.hidden, bufs.cap
        self.args = a

    def launch(self, pdl: bool = False, stream=None):
        lib = _ext.require()
        self.heap.level_launch_counters(_ext.SITE_A2A_COMBINE, self.grid)
        _ext.check(lib.mcb_launch_a2a_combine(C.byref(self.heap.ctx()), C.byref(self.args), self.grid,
                                              self.threads, int(pdl), _ext.stream_handle(stream)),
                   "a2a_combine")


def a2a_decode_step(heap, d: A2ADispatchPlan, c: A2ACombinePlan, num_layers: int, pdl: bool = False, stream=None):
    lib = _ext.require()
    heap.level_launch_counters(_ext.SITE_A2A_COMBINE, d.grid)
    _ext.check(lib.mcb_a2a_decode_step(C.byref(heap.ctx()), C.byref(d.args), C.byref(c.args), int(num_layers),
                                       d.grid, d.threads, int(pdl), _ext.stream_handle(stream)),
               "a2a_decode_step")


def dequant_e4m3_1x128(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """[rows, H] e4m3 bytes + [rows, H/128] fp32 scales -> bf16 (host-layer helper)."""
    f = q.view(torch.float8_e4m3fn).to(torch.float32)
    return (f.view(*scale.shape, 128) * scale.unsqueeze(-1)).view(q.shape).to(torch.bfloat16)
