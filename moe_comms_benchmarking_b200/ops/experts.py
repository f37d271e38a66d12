"""Expert path: routing of gathered tokens, grouped SwiGLU GEMMs on tcgen05, and the combine
that pre-sums a token's local expert outputs and reduce-scatters across ranks.

The reference's expert is the identity (bench_nvls.py:109-112, bench_nccl.py:106-109); these
plans are what turns the dense transport into a full expert-parallel MoE layer:

    gathered tokens --RoutePlan--> pair lists, row tiles
                    --GroupedGemmPlan(FC1)--> act = silu(x Wg^T) * (x Wu^T)      (token gather fused)
                    --GroupedGemmPlan(FC2)--> y = prob * (act Wd^T)
                    --ExpertCombinePlan--> out[t] = sum over ranks and local pairs of y
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _ext
from .dense import _check_heap_tensor
from ..parallel.symm_heap import HeapTensor, SymmetricHeap

NUM_SMS = 148
BLOCK_M = 128


def _swizzle(t: torch.Tensor) -> torch.Tensor:
    """``t[..., 8 (row % 8), 8 (16-byte chunk), 8 values]`` -> chunk c of row r moved to position c ^ r (its own inverse)."""
    r = torch.arange(8, device=t.device).view(8, 1)
    c = torch.arange(8, device=t.device).view(1, 8) ^ r
    return t[..., r, c, :]


def pack_weight_tiles(w: torch.Tensor) -> torch.Tensor:
    """``[E, R, K]`` row-major bf16 -> ``[E, R/128, K/64, 128, 64]``: every (128-row, 64-column) tile as 16 KB of
    contiguous memory in the K-major shared-memory image with 128-byte swizzle (16-byte chunk c of row r of a
    tile is stored at chunk position c ^ (r % 8)), the tiles of a 128-row block one after the other."""
    E, R, K = w.shape
    if R % 128 or K % 64:
        raise ValueError("rows must be a multiple of 128 and columns a multiple of 64")
    t = w.view(E, R // 128, 16, 8, K // 64, 8, 8).permute(0, 1, 4, 2, 3, 5, 6)      # [E, RB, KB, 16, row % 8, chunk, 8]
    return _swizzle(t).contiguous().view(E, R // 128, K // 64, 128, 64)


def unpack_weight_tiles(p: torch.Tensor) -> torch.Tensor:
    """Inverse of ``pack_weight_tiles``."""
    E, RB, KB = p.shape[:3]
    t = _swizzle(p.view(E, RB, KB, 16, 8, 8, 8))                                    # [E, RB, KB, 16, row % 8, chunk, 8]
    return t.permute(0, 1, 3, 4, 2, 5, 6).contiguous().view(E, RB * 128, KB * 64)


class ExpertWeights:
    """bf16 weights of this rank's experts: random N(0, std^2), generated as gate/up ``[E_loc, 2*I, H]`` (gate rows
    first) and down ``[E_loc, H, I]``, kept in the form the kernels stream:

    * ``layout="packed"`` (default), for the weights-as-M FFN kernel: the gate/up rows interleaved (row ``2i`` =
      gate row ``i``, row ``2i + 1`` = up row ``i``, so a 128-row block holds 64 finished activations) and both
      matrices packed tile by tile into their shared-memory image (``pack_weight_tiles``): ``w1``, ``w2``;
    * ``layout="split"``, for the tokens-as-rows GEMM kernels: row-major matrices with TMA tensor maps.

    ``w_gate_up`` / ``w_down`` always return the plain row-major matrices (unpacked on demand), which is what the
    CPU oracle takes."""

    def __init__(self, num_local_experts: int, hidden: int, intermediate: int, device, seed: int = 0, std: float = 0.02,
                 layout: str = "packed"):
        if hidden % 256 or intermediate % 128:
            raise ValueError("hidden must be a multiple of 256 and intermediate a multiple of 128")
        if layout not in ("packed", "split"):
            raise ValueError(f"unknown weight layout {layout!r}")
        g = torch.Generator(device=device).manual_seed(seed)
        self.num_local_experts, self.hidden, self.intermediate = num_local_experts, hidden, intermediate
        self.layout = layout
        split = (torch.randn(num_local_experts, 2 * intermediate, hidden, device=device, generator=g,
                             dtype=torch.float32) * std).to(torch.bfloat16)
        down = (torch.randn(num_local_experts, hidden, intermediate, device=device, generator=g,
                            dtype=torch.float32) * std).to(torch.bfloat16)
        if layout == "packed":
            self.w1 = pack_weight_tiles(self.interleave(split))
            self.w2 = pack_weight_tiles(down)
            del split, down
        else:
            self.w1, self.w2 = split, down
            self.map_w1 = make_weight_tmap(self.w1.view(-1, hidden))
            self.map_down = make_weight_tmap(self.w2.view(-1, intermediate))

    @staticmethod
    def interleave(split: torch.Tensor) -> torch.Tensor:
        """``[E, 2I, H]`` gate rows then up rows -> row 2i = gate i, row 2i + 1 = up i."""
        E, two_i, H = split.shape
        return split.view(E, 2, two_i // 2, H).transpose(1, 2).contiguous().view(E, two_i, H)

    @property
    def w_gate_up(self) -> torch.Tensor:
        if self.layout == "split":
            return self.w1
        il = unpack_weight_tiles(self.w1)
        E, two_i, H = il.shape
        return il.view(E, two_i // 2, 2, H).transpose(1, 2).contiguous().view(E, two_i, H)

    @property
    def w_down(self) -> torch.Tensor:
        return self.w2 if self.layout == "split" else unpack_weight_tiles(self.w2)

    @property
    def map_gate_up(self):
        if self.layout != "split":
            raise ValueError("the tokens-as-rows GEMM kernels need ExpertWeights(layout='split')")
        return self.map_w1

    def bytes(self) -> int:
        return (self.w1.numel() + self.w2.numel()) * 2


def make_weight_tmap(w2d: torch.Tensor):
    """128-byte tensor map (kept in 64-byte aligned host memory) over a row-major bf16 matrix."""
    if w2d.dtype != torch.bfloat16 or w2d.dim() != 2 or not w2d.is_contiguous():
        raise ValueError("weights must be a contiguous 2-D bf16 tensor")
    raw = (C.c_uint8 * 192)()
    addr = (C.addressof(raw) + 63) & ~63
    lib = _ext.require()
    _ext.check(lib.mcb_make_weight_tmap(C.c_void_p(addr), C.c_void_p(w2d.data_ptr()), C.c_uint64(w2d.shape[0]),
                                        C.c_uint64(w2d.shape[1])), "make_weight_tmap")
    return (raw, addr)     # keep `raw` alive; `addr` is what launches take


class RouteBuffers:
    """Device buffers written by the routing kernel and read by the GEMMs and the combine."""

    def __init__(self, max_tokens: int, topk: int, num_local_experts: int, device):
        self.max_tokens, self.topk, self.E = max_tokens, topk, num_local_experts
        self.max_pairs = max_tokens * min(topk, num_local_experts)
        self.max_tiles = num_local_experts + self.max_pairs // BLOCK_M + 1
        i32 = dict(dtype=torch.int32, device=device)
        self.expert_count = torch.zeros(num_local_experts, **i32)
        self.expert_cursor = torch.zeros(num_local_experts, **i32)
        self.expert_offset = torch.zeros(num_local_experts + 1, **i32)
        self.pair_token = torch.zeros(max(self.max_pairs, 1), **i32)
        self.pair_prob = torch.zeros(max(self.max_pairs, 1), dtype=torch.float32, device=device)
        self.pair_pos = torch.full((max_tokens, topk), -1, **i32)
        self.tile_expert = torch.zeros(self.max_tiles, **i32)
        self.tile_row0 = torch.zeros(self.max_tiles, **i32)
        self.tile_rows = torch.zeros(self.max_tiles, **i32)
        self.num_m_tiles = torch.zeros(1, **i32)
        self.sync = torch.zeros(4, **i32)
        self.max_rows = torch.zeros(1, **i32)            # largest pair count of one expert
        self.ffn_done = torch.zeros(num_local_experts, **i32)   # gate/up blocks finished per expert (fused FFN)


class RoutePlan:
    def __init__(self, bufs: RouteBuffers, topk_idx: torch.Tensor, topk_w: torch.Tensor | None, num_tokens: torch.Tensor,
                 expert_begin: int, status: torch.Tensor | None = None, grid: int = 32, timeout_s: float = 2.0):
        if topk_idx.dtype != torch.int64 or topk_idx.dim() != 2 or topk_idx.shape[1] != bufs.topk:
            raise ValueError("topk_idx must be int64 [tokens, topk]")
        if topk_idx.shape[0] < bufs.max_tokens:
            raise ValueError("topk_idx holds fewer rows than max_tokens")
        if num_tokens.dtype != torch.int32:
            raise ValueError("num_tokens must be an int32 device scalar")
        if not (1 <= grid <= 128):
            raise ValueError("routing grid must be in [1, 128] (its blocks wait on one another)")
        self.bufs, self.grid = bufs, grid
        self._keep = (topk_idx, topk_w, num_tokens, status)
        a = _ext.McbRouteArgs()
        a.topk_idx, a.topk_w, a.num_tokens = topk_idx.data_ptr(), _ext.ptr(topk_w), num_tokens.data_ptr()
        a.topk, a.expert_begin, a.num_local_experts, a.max_tokens = bufs.topk, int(expert_begin), bufs.E, bufs.max_tokens
        for f in ("expert_count", "expert_cursor", "expert_offset", "pair_token", "pair_prob", "pair_pos",
                  "tile_expert", "tile_row0", "tile_rows", "num_m_tiles", "sync", "max_rows", "ffn_done"):
            setattr(a, f, getattr(bufs, f).data_ptr())
        a.max_pairs, a.max_tiles = bufs.max_pairs, bufs.max_tiles
        a.status, a.timeout_ns = _ext.ptr(status), int(timeout_s * 1e9)
        self.args = a

    def launch(self, pdl: bool = False, stream=None):
        lib = _ext.require()
        _ext.check(lib.mcb_launch_route(C.byref(self.args), self.grid, int(pdl), _ext.stream_handle(stream)), "route")


class GroupedGemmPlan:
    """One grouped GEMM over the row tiles of ``route``.  ``mode`` FC1: ``a`` = gathered hidden
    ``[T, H]`` gathered through ``pair_token``, ``out`` = act ``[P, I]``.  FC2: ``a`` = act
    (identity rows), ``out`` = y ``[P, H]`` scaled by ``pair_prob``."""

    def __init__(self, mode: int, tmap, route: RouteBuffers, a: torch.Tensor, out: torch.Tensor, n_total: int,
                 k_total: int, status: torch.Tensor | None = None, grid: int = NUM_SMS, timeout_s: float = 2.0):
        if a.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or not a.is_contiguous() or not out.is_contiguous():
            raise ValueError("A and out must be contiguous bf16")
        if a.shape[-1] != k_total:
            raise ValueError(f"A rows hold {a.shape[-1]} values, k_total is {k_total}")
        n_out = n_total // 2 if mode == _ext.GEMM_FC1 else n_total
        if out.shape[-1] != n_out or out.shape[0] < route.max_pairs:
            raise ValueError("out must be [max_pairs, n_out]")
        if k_total % 64 or n_total % 256:
            raise ValueError("k_total must be a multiple of 64 and n_total of 256")
        self.mode, self.tmap, self.grid = mode, tmap, grid
        self._keep = (route, a, out, status)
        g = _ext.McbGemmArgs()
        g.a_base, g.a_row_bytes = a.data_ptr(), k_total * 2
        g.row_index = route.pair_token.data_ptr() if mode == _ext.GEMM_FC1 else 0
        g.row_scale = route.pair_prob.data_ptr() if mode == _ext.GEMM_FC2 else 0
        g.out, g.out_row_bytes = out.data_ptr(), n_out * 2
        g.tile_expert, g.tile_row0 = route.tile_expert.data_ptr(), route.tile_row0.data_ptr()
        g.tile_rows, g.num_m_tiles = route.tile_rows.data_ptr(), route.num_m_tiles.data_ptr()
        g.n_total, g.k_total = int(n_total), int(k_total)
        g.status, g.timeout_ns = _ext.ptr(status), int(timeout_s * 1e9)
        self.args = g

    def launch(self, pdl: bool = False, stream=None):
        lib = _ext.require()
        _ext.check(lib.mcb_launch_grouped_gemm(C.c_void_p(self.tmap[1]), C.byref(self.args), self.mode, self.grid,
                                               int(pdl), _ext.stream_handle(stream)), "grouped_gemm")


class ExpertCombinePlan:
    def __init__(self, heap: SymmetricHeap, y: torch.Tensor, route: RouteBuffers, partial: HeapTensor, out: torch.Tensor,
                 n_local: torch.Tensor, step_meta: torch.Tensor, cap: int, grid: int = NUM_SMS, threads: int = 512,
                 site: int = _ext.SITE_FUSED_FC2):
        hidden = y.shape[-1]
        if y.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or hidden % 8:
            raise ValueError("y and out must be bf16 with hidden a multiple of 8")
        _check_heap_tensor(heap, partial, "combine partial sums")
        rows = cap * heap.world
        two = partial.tensor.dim() == 3         # [2, cap * world, hidden]: alternate copies, layer by layer
        if (two and (partial.tensor.shape[0] != 2 or partial.tensor.shape[1] < rows)) or partial.nbytes < rows * hidden * 2:
            raise ValueError("partial-sum buffer must be [cap * world, hidden] or [2, cap * world, hidden]")
        self.heap, self.grid, self.threads = heap, grid, threads
        self._keep = (y, route, partial, out, n_local, step_meta)
        a = _ext.McbCombineArgs()
        a.y, a.pair_pos, a.partial_off, a.out = y.data_ptr(), route.pair_pos.data_ptr(), partial.offset, out.data_ptr()
        a.n_local, a.step_meta = n_local.data_ptr(), step_meta.data_ptr()
        a.hidden, a.topk, a.cap, a.site = hidden, route.topk, int(cap), int(site)
        a.partial_par_stride = partial.nbytes // 2 if two else 0
        self.args = a

    def launch(self, pdl: bool = False, stream=None):
        lib = _ext.require()
        _ext.check(lib.mcb_launch_combine(C.byref(self.heap.ctx()), C.byref(self.args), self.grid, self.threads,
                                          int(pdl), _ext.stream_handle(stream)), "expert_combine")


class Fc2CombinePlan:
    """FC2 grouped GEMM and the cross-rank combine as ONE cooperative kernel launch
    (``fc2_combine_kernel``): GEMM tiles, grid-wide barrier, local pre-sum, cross-GPU barrier,
    switch-side reduction.  Built from the two stand-alone plans so both forms share arguments."""

    def __init__(self, heap: SymmetricHeap, fc2: GroupedGemmPlan, combine: ExpertCombinePlan, grid: int = NUM_SMS):
        if fc2.mode != _ext.GEMM_FC2:
            raise ValueError("Fc2CombinePlan needs an FC2 plan")
        if not (1 <= grid <= NUM_SMS):
            raise ValueError("the fused kernel needs all its blocks resident at once: grid <= number of SMs")
        self.heap, self.fc2, self.combine, self.grid = heap, fc2, combine, grid

    def launch(self, pdl: bool = False, stream=None):
        lib = _ext.require()
        _ext.check(lib.mcb_launch_fc2_combine(C.c_void_p(self.fc2.tmap[1]), C.byref(self.fc2.args),
                                              C.byref(self.heap.ctx()), C.byref(self.combine.args), self.grid,
                                              int(pdl), _ext.stream_handle(stream)), "fc2_combine")


class DispatchRouteFc1Plan:
    """All-gather-V dispatch, routing and the FC1 grouped GEMM as ONE cooperative kernel launch
    (``dispatch_route_fc1_kernel``): multicast push + cross-GPU barrier (or flagged packets),
    grid-wide barrier, routing, grid-wide barrier, tcgen05 GEMM that gathers token rows from the
    buffer the peers just filled.  Built from the three stand-alone plans."""

    def __init__(self, heap: SymmetricHeap, agv, route: RoutePlan, fc1: GroupedGemmPlan, grid: int = NUM_SMS):
        if fc1.mode != _ext.GEMM_FC1:
            raise ValueError("DispatchRouteFc1Plan needs an FC1 plan")
        if not (1 <= grid <= NUM_SMS):
            raise ValueError("the fused kernel needs all its blocks resident at once: grid <= number of SMs")
        self.heap, self.agv, self.route, self.fc1, self.grid = heap, agv, route, fc1, grid

    def launch(self, pdl: bool = False, stream=None):
        lib = _ext.require()
        _ext.check(lib.mcb_launch_dispatch_route_fc1(C.c_void_p(self.fc1.tmap[1]), C.byref(self.fc1.args),
                                                     C.byref(self.heap.ctx()), C.byref(self.agv.args),
                                                     C.byref(self.route.args), self.grid, int(pdl),
                                                     _ext.stream_handle(stream)), "dispatch_route_fc1")


def _aligned_layer_args(count: int):
    """``count`` zeroed McbLayerArgs in 64-byte aligned host memory: (keep-alive buffer, address, stride)."""
    stride = _ext.layer_args_size()
    raw = (C.c_uint8 * (stride * count + 64))()
    addr = (C.addressof(raw) + 63) & ~63
    return raw, addr, stride


class ExpertFfnPlan:
    """Gate/up + SwiGLU + down over the pair lists of ``route`` as ONE persistent launch
    (``expert_ffn_kernel``): weights are the M = 128 operand, an expert's tokens the small N."""

    def __init__(self, weights: ExpertWeights, route: RouteBuffers, x: torch.Tensor, act: torch.Tensor, y: torch.Tensor,
                 status: torch.Tensor | None = None, grid: int = NUM_SMS, timeout_s: float = 2.0):
        H, I = weights.hidden, weights.intermediate
        if weights.layout != "packed":
            raise ValueError("the FFN kernel streams the packed weight layout")
        for t, cols, what in ((x, H, "x"), (act, I, "act"), (y, H, "y")):
            if t.dtype != torch.bfloat16 or not t.is_contiguous() or t.shape[-1] != cols:
                raise ValueError(f"{what} must be contiguous bf16 with {cols} columns")
        if act.shape[0] < route.max_pairs or y.shape[0] < route.max_pairs:
            raise ValueError("act and y must hold max_pairs rows")
        if not (1 <= grid <= NUM_SMS):
            raise ValueError("down blocks wait for gate/up blocks of other CTAs: grid <= number of SMs")
        self.weights, self.grid = weights, grid
        self._keep = (route, x, act, y, status)
        a = _ext.McbFfnArgs()
        a.x, a.x_row_bytes = x.data_ptr(), H * 2
        a.pair_token, a.pair_prob = route.pair_token.data_ptr(), route.pair_prob.data_ptr()
        a.expert_offset, a.max_rows = route.expert_offset.data_ptr(), route.max_rows.data_ptr()
        a.act, a.y, a.ffn_done = act.data_ptr(), y.data_ptr(), route.ffn_done.data_ptr()
        a.num_local_experts, a.hidden, a.intermediate = weights.num_local_experts, H, I
        a.status, a.timeout_ns = _ext.ptr(status), int(timeout_s * 1e9)
        a.w1, a.w2 = weights.w1.data_ptr(), weights.w2.data_ptr()
        self.args = a

    def launch(self, pdl: bool = False, stream=None):
        lib = _ext.require()
        _ext.check(lib.mcb_launch_expert_ffn(C.byref(self.args), self.grid, int(pdl), _ext.stream_handle(stream)),
                   "expert_ffn")


class MoeLayerPlan:
    """One whole MoE layer per launch (``moe_layer_kernel``: dispatch, routing, experts, combine), for
    one or several weight sets; ``launch(s)`` runs the layer with set ``s``, ``decode_step(n)`` issues the
    count exchange and ``n`` layers natively (layer l uses set l % sets)."""

    def __init__(self, heap: SymmetricHeap, agv, route: RoutePlan, ffns: list[ExpertFfnPlan], combine: ExpertCombinePlan,
                 meta, grid: int = NUM_SMS, trace: bool = False):
        if not (1 <= grid <= NUM_SMS):
            raise ValueError("the layer kernel needs all its blocks resident at once: grid <= number of SMs")
        self.heap, self.agv, self.route, self.ffns, self.combine, self.meta, self.grid = heap, agv, route, ffns, combine, meta, grid
        # phase trace: 8 global-timer stamps of block 0 of the LAST layer launched (see phase_times)
        self.trace = torch.zeros(8, dtype=torch.int64, device=heap.device) if trace else None
        self._raw, self._addr, self._stride = _aligned_layer_args(len(ffns))
        self._ctx_version = None
        self._fill()

    def _fill(self):
        ctx = self.heap.ctx()
        for s, f in enumerate(self.ffns):
            p = _ext.McbLayerArgs.from_address(self._addr + s * self._stride)
            C.memmove(C.addressof(p.ctx), C.addressof(ctx), C.sizeof(_ext.McbCtx))
            C.memmove(C.addressof(p.agv), C.addressof(self.agv.args), C.sizeof(_ext.McbAgvArgs))
            C.memmove(C.addressof(p.route), C.addressof(self.route.args), C.sizeof(_ext.McbRouteArgs))
            C.memmove(C.addressof(p.ffn), C.addressof(f.args), C.sizeof(_ext.McbFfnArgs))
            C.memmove(C.addressof(p.cmb), C.addressof(self.combine.args), C.sizeof(_ext.McbCombineArgs))
            p.trace = self.trace.data_ptr() if self.trace is not None else None
        self._ctx_version = id(ctx)

    def _sync_ctx(self):
        if self._ctx_version != id(self.heap.ctx()):      # the heap's context was rebuilt (e.g. a new timeout)
            self._fill()

    PHASES = ("dispatch", "grid barrier", "routing", "grid barrier", "experts", "grid barrier", "combine")

    def phase_times(self):
        """[(phase, microseconds)] of the last layer launched, as block 0 saw it (needs ``trace=True``; read after
        a synchronize)."""
        if self.trace is None:
            raise RuntimeError("built without trace=True")
        t = self.trace.cpu().tolist()
        return [(name, (t[i + 1] - t[i]) / 1e3) for i, name in enumerate(self.PHASES)]

    def args(self, s: int = 0) -> "_ext.McbLayerArgs":
        return _ext.McbLayerArgs.from_address(self._addr + s * self._stride)

    def launch(self, s: int = 0, pdl: bool = False, stream=None):
        lib = _ext.require()
        self._sync_ctx()
        _ext.check(lib.mcb_launch_moe_layer(C.c_void_p(self._addr + s * self._stride), self.grid, int(pdl),
                                            _ext.stream_handle(stream)), "moe_layer")

    def decode_step(self, num_layers: int, pdl: bool = False, stream=None):
        lib = _ext.require()
        self._sync_ctx()
        _ext.check(lib.mcb_moe_decode_step(C.byref(self.heap.ctx()), C.byref(self.meta.args), C.c_void_p(self._addr),
                                           len(self.ffns), int(num_layers), self.grid, int(pdl),
                                           _ext.stream_handle(stream)), "moe_decode_step")
