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


def a2a_meta_row_bytes(topk: int) -> int:
    """Bytes of a packed metadata row of the step kernel: {stamp, token, (expert id, weight) x topk}, in 16-byte chunks."""
    return (8 + 8 * topk + 15) // 16 * 16


def a2a_ll_words(hidden: int, topk: int, fp8: bool):
    """8-byte words per token of the packet-mode staging areas: (dispatch incl. the header word, combine)."""
    xdata = hidden // 8 if fp8 else hidden // 4
    scales = hidden // 256 if fp8 else 0
    return 1 + xdata + scales + a2a_meta_row_bytes(topk) // 8, hidden // 4


def a2a_ll_specs(world: int, cap: int, hidden: int, topk: int, fp8: bool, ll_rows: int):
    """Heap regions of packet mode: dispatch staging, combine staging, per-(block, source) credit words."""
    if ll_rows <= 0 or world == 1:
        return []
    src_rows = min(cap, ll_rows)
    xw, yw = a2a_ll_words(hidden, topk, fp8)
    return [([2 * world * src_rows * xw * 16], torch.uint8), ([2 * world * src_rows * yw * 16], torch.uint8),
            ([_ext.MAX_BLOCKS * _ext.MAX_RANKS * 4], torch.uint8)]


class A2AStepBuffers:
    """Heap buffers of the persistent all-to-all step kernel, double buffered by layer parity:
    ``recv_x [2, world, cap, hidden]`` (bf16, or e4m3 bytes with ``recv_scale [2, world, cap, hidden/128]``),
    ``recv_meta [2, world, cap, meta_row_bytes]`` and the expert outputs ``y`` (the received rows themselves
    for the identity expert in bf16).  A token's slot on every destination is its own index.  With
    ``ll_rows > 0`` the packet-mode staging areas and credit words are allocated too (e4m3 packet mode needs
    ``hidden % 256 == 0``; otherwise the kernel stays on the barrier path)."""

    def __init__(self, heap: SymmetricHeap, cap: int, hidden: int, topk: int, fp8: bool, prefix: str = "a2as",
                 ll_rows: int = 0):
        w = heap.world
        self.cap, self.hidden, self.topk, self.fp8 = cap, hidden, topk, fp8
        self.meta_row_bytes = a2a_meta_row_bytes(topk)
        self.ll_rows = int(ll_rows) if w > 1 and hidden % 4 == 0 else 0
        self.ll_x = self.ll_y = self.credits = None
        if self.ll_rows > 0:
            sx, sy, sc = a2a_ll_specs(w, cap, hidden, topk, fp8, self.ll_rows)
            self.ll_x = heap.alloc(f"{prefix}_ll_x", sx[0], torch.uint8)
            self.ll_y = heap.alloc(f"{prefix}_ll_y", sy[0], torch.uint8)
            self.credits = heap.alloc(f"{prefix}_credit", sc[0], torch.uint8)
            self.credits.tensor.zero_()
        if hidden % 8 or (fp8 and hidden % 128):
            raise ValueError("hidden must be a multiple of 8 (128 with fp8 dispatch)")
        if fp8:
            self.recv_x = heap.alloc(f"{prefix}_recv_x8", [2, w, cap, hidden], torch.uint8)
            self.recv_scale = heap.alloc(f"{prefix}_recv_scale", [2, w, cap, hidden // 128], torch.float32)
            self.y = heap.alloc(f"{prefix}_y", [2, w, cap, hidden], torch.bfloat16)
        else:
            self.recv_x = heap.alloc(f"{prefix}_recv_x", [2, w, cap, hidden], torch.bfloat16)
            self.recv_scale = None
            self.y = self.recv_x
        self.recv_meta = heap.alloc(f"{prefix}_recv_meta", [2, w, cap, self.meta_row_bytes], torch.uint8)

    @staticmethod
    def specs(world: int, cap: int, hidden: int, topk: int, fp8: bool, ll_rows: int = 0):
        s = [([2, world, cap, a2a_meta_row_bytes(topk)], torch.uint8)]
        s += a2a_ll_specs(world, cap, hidden, topk, fp8, ll_rows if hidden % 4 == 0 else 0)
        if fp8:
            s += [([2, world, cap, hidden], torch.uint8), ([2, world, cap, hidden // 128], torch.float32),
                  ([2, world, cap, hidden], torch.bfloat16)]
        else:
            s += [([2, world, cap, hidden], torch.bfloat16)]
        return s

    def meta_fields(self, par: int, src: int, rows: int):
        """(stamp int32 [rows], token int32 [rows], expert ids int32 [rows, topk], weights fp32 [rows, topk]) of the
        metadata rows received from ``src`` in parity ``par``."""
        raw = self.recv_meta.tensor[par, src, :rows]
        words = raw.view(torch.int32).view(rows, -1)
        ids = words[:, 2:2 + 2 * self.topk:2]
        wts = words[:, 3:3 + 2 * self.topk:2].view(torch.float32) if rows else words[:, 3:3].view(torch.float32)
        return words[:, 0], words[:, 1], ids, wts


class A2AStepPlan:
    """One whole decode step of the all-to-all dispatcher as ONE persistent launch (``a2a_step_kernel``)."""

    def __init__(self, heap: SymmetricHeap, bufs: A2AStepBuffers, x, topk_idx, topk_w, out, n_local, step_meta,
                 num_experts: int, num_layers: int, grid: int = DEFAULT_GRID, threads: int = DEFAULT_THREADS,
                 state: torch.Tensor | None = None):
        _check_grid(grid, threads)
        if x.dtype != torch.bfloat16 or x.dim() != 2 or x.shape[1] != bufs.hidden or not x.is_contiguous():
            raise ValueError("x must be contiguous bf16 [rows, hidden]")
        if topk_idx.dtype != torch.int64 or topk_idx.shape[1] != bufs.topk or not topk_idx.is_contiguous():
            raise ValueError("topk_idx must be contiguous int64 [rows, topk]")
        if topk_w is not None and (topk_w.dtype != torch.float32 or not topk_w.is_contiguous()):
            raise ValueError("topk_w must be contiguous fp32 [rows, topk]")
        if out.dtype != torch.bfloat16 or out.shape[1] != bufs.hidden or min(x.shape[0], topk_idx.shape[0], out.shape[0]) < bufs.cap:
            raise ValueError("input and output buffers must hold `cap` rows of `hidden` bf16 values")
        if num_experts % heap.world:
            raise ValueError("num_experts must be divisible by the world size")
        if step_meta.dtype != torch.int32 or step_meta.numel() < 8:
            raise ValueError("step_meta must be int32[8]")
        for name in ("recv_x", "recv_meta", "y"):
            _check_heap_tensor(heap, getattr(bufs, name), name)
        if state is None:
            state = torch.zeros(_ext.STEP_STATE_WORDS, dtype=torch.int32, device=heap.device)
        self.heap, self.bufs, self.grid, self.threads, self.state = heap, bufs, grid, threads, state
        self._keep = (x, topk_idx, topk_w, out, n_local, step_meta)
        a = _ext.McbA2AStepArgs()
        a.x, a.topk_idx, a.topk_w, a.out = x.data_ptr(), topk_idx.data_ptr(), _ext.ptr(topk_w), out.data_ptr()
        a.n_local = n_local.data_ptr()
        a.recv_x_off, a.x_par_stride = bufs.recv_x.offset, bufs.recv_x.nbytes // 2
        if bufs.recv_scale is not None:
            a.recv_scale_off, a.scale_par_stride = bufs.recv_scale.offset, bufs.recv_scale.nbytes // 2
        a.recv_meta_off, a.meta_par_stride = bufs.recv_meta.offset, bufs.recv_meta.nbytes // 2
        a.y_off, a.y_par_stride = bufs.y.offset, bufs.y.nbytes // 2
        a.meta_row_bytes, a.hidden, a.topk, a.num_experts = bufs.meta_row_bytes, bufs.hidden, bufs.topk, int(num_experts)
        a.cap, a.fp8, a.num_layers = bufs.cap, int(bufs.fp8), int(num_layers)
        a.step_meta, a.counts_off, a.state = step_meta.data_ptr(), heap.a2a_counts_off, state.data_ptr()
        if bufs.ll_rows > 0:
            for name in ("ll_x", "ll_y", "credits"):
                _check_heap_tensor(heap, getattr(bufs, name), name)
            a.ll_rows, a.ll_src_rows = bufs.ll_rows, min(bufs.cap, bufs.ll_rows)
            a.ll_x_off, a.ll_y_off, a.credit_off = bufs.ll_x.offset, bufs.ll_y.offset, bufs.credits.offset
        self.args = a

    def launch(self, pdl: bool = False, stream=None):
        lib = _ext.require()
        _ext.check(lib.mcb_launch_a2a_step(C.byref(self.heap.ctx()), C.byref(self.args), self.grid, self.threads,
                                           int(pdl), _ext.stream_handle(stream)), "a2a_step")


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
