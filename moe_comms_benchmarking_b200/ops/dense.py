"""Dense expert-parallel collectives on the symmetric heap: token-count metadata,
variable all-gather (dispatch) and variable reduce-scatter (combine), plus the
uniform-count all-gather / reduce-scatter built on the same kernels.

API surface of the reference's op layer (nvls/torch_symm_triton/__init__.py:3-10,
nvls/metadata.py:111-139): ``fused_metadata_update``, ``multimem_all_gather_v``,
``multimem_all_gatherv_3tensor``, ``multimem_reduce_scatter_v``, ``multimem_all_gather``,
``multimem_all_gather_fused`` and ``multimem_reduce_scatter`` map to ``MetadataPlan``,
``AllGatherVPlan`` (1 to 4 tensors), ``ReduceScatterVPlan`` and the ``uniform_*`` helpers.

A *plan* owns the C argument block of one kernel; building it validates shapes, alignment
and capacities on the host (the substitute for a device-side sanitizer), launching it is one
ctypes call.  All per-step sizes are read by the kernels from device memory, so a plan (and
a CUDA graph that contains it) stays valid while the batch changes.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _ext
from ..parallel.symm_heap import HeapTensor, SymmetricHeap

DEFAULT_GRID = 148      # one block per B200 SM
DEFAULT_THREADS = 512


def _check_heap_tensor(heap: SymmetricHeap, ht: HeapTensor, what: str):
    if ht.offset < 0 or ht.offset + ht.nbytes > heap.nbytes:
        raise ValueError(f"{what}: heap range [{ht.offset}, {ht.offset + ht.nbytes}) outside the heap")
    if ht.offset % 16:
        raise ValueError(f"{what}: heap offset {ht.offset} is not 16-byte aligned")


def _row_bytes(t: torch.Tensor) -> int:
    if t.dim() != 2:
        raise ValueError("expected a 2-D [rows, cols] tensor")
    if not t.is_contiguous():
        raise ValueError("expected a contiguous tensor")
    return t.shape[1] * t.element_size()


def _check_grid(grid: int, threads: int):
    if not (1 <= grid <= _ext.MAX_BLOCKS):
        raise ValueError(f"grid {grid} outside [1, {_ext.MAX_BLOCKS}]")
    if not (32 <= threads <= 512) or threads % 32:
        raise ValueError(f"threads {threads} must be a multiple of 32 in [32, 512]")


def agv_ll_stage_bytes(ll_rows: int, row_bytes: list[int]) -> int:
    """Staging bytes of the low-latency all-gather: 2 parities x ll_rows rows (all ranks together)
    x one 16-byte packet per 8 bytes of row."""
    return 2 * ll_rows * sum(rb // 8 for rb in row_bytes) * 16


def rsv_ll_stage_bytes(world: int, ll_rows: int, cap: int, row_bytes: int) -> int:
    """Staging bytes of the low-latency reduce-scatter: 2 parities x world sources x
    min(cap, ll_rows) rows (one rank may own every row of a small step)."""
    return 2 * world * min(cap, ll_rows) * (row_bytes // 8) * 16


class MetadataPlan:
    """counts -> ``step_meta = [valid, offset, max, epoch]`` (int32, local device tensor)."""

    def __init__(self, heap: SymmetricHeap, n_local: torch.Tensor, step_meta: torch.Tensor, cap: int):
        if n_local.dtype != torch.int32 or n_local.numel() != 1:
            raise ValueError("n_local must be an int32 scalar tensor on the device")
        if step_meta.dtype != torch.int32 or step_meta.numel() < 4:
            raise ValueError("step_meta must be int32[4]")
        self.heap, self.n_local, self.step_meta = heap, n_local, step_meta
        a = _ext.McbMetaArgs()
        a.n_local = n_local.data_ptr()
        a.counts_off = heap.counts_off
        a.step_meta = step_meta.data_ptr()
        a.cap = int(cap)
        self.args = a

    def launch(self, pdl: bool = False, stream=None):
        lib = _ext.require()
        _ext.check(lib.mcb_launch_metadata(C.byref(self.heap.ctx()), C.byref(self.args), int(pdl),
                                           _ext.stream_handle(stream)), "metadata")


class AllGatherVPlan:
    """Gather ``srcs[i][:n]`` of every rank into packed ``dsts[i]`` at row offset
    ``step_meta[1]``.  1 to 4 tensors per launch; rows must be multiples of 4 bytes
    (16-byte rows use 128-bit accesses, 8-byte rows 64-bit)."""

    def __init__(self, heap: SymmetricHeap, dsts, srcs, n_local, step_meta, cap: int,
                 site: int = _ext.SITE_AGV, grid: int = DEFAULT_GRID, threads: int = DEFAULT_THREADS,
                 ll_stage: HeapTensor | None = None, ll_rows: int = 0):
        if not (1 <= len(srcs) <= _ext.MAX_TENSORS) or len(srcs) != len(dsts):
            raise ValueError(f"need 1..{_ext.MAX_TENSORS} (dst, src) pairs")
        _check_grid(grid, threads)
        self.heap, self.grid, self.threads = heap, grid, threads
        self._keep = (list(dsts), list(srcs), n_local, step_meta)
        a = _ext.McbAgvArgs()
        gcap = cap * heap.world
        for i, (d, s) in enumerate(zip(dsts, srcs)):
            rb = _row_bytes(s)
            _check_heap_tensor(heap, d, f"all_gather_v dst[{i}]")
            if rb % 4:
                raise ValueError(f"row of tensor {i} is {rb} bytes; must be a multiple of 4")
            if d.tensor.dtype != s.dtype or d.tensor.shape[1:] != s.shape[1:]:
                raise ValueError(f"tensor {i}: dst/src dtype or row shape differ")
            if s.shape[0] < cap:
                raise ValueError(f"tensor {i}: source holds {s.shape[0]} rows, capacity is {cap}")
            if d.nbytes < gcap * rb:
                raise ValueError(f"tensor {i}: gathered buffer too small for {gcap} rows of {rb} bytes")
            if s.data_ptr() % 16:
                raise ValueError(f"tensor {i}: source is not 16-byte aligned")
            a.src[i] = s.data_ptr()
            a.dst_off[i] = d.offset
            a.row_bytes[i] = rb
        a.num_tensors, a.cap, a.site = len(srcs), int(cap), int(site)
        a.n_local, a.step_meta = n_local.data_ptr(), step_meta.data_ptr()
        if ll_stage is not None and ll_rows > 0:
            need = agv_ll_stage_bytes(ll_rows, [_row_bytes(s) for s in srcs])
            _check_heap_tensor(heap, ll_stage, "all_gather_v low-latency staging")
            if ll_stage.nbytes < need:
                raise ValueError(f"low-latency staging holds {ll_stage.nbytes} bytes, {need} needed")
            a.ll_off, a.ll_rows = ll_stage.offset, int(ll_rows)
            self._keep += (ll_stage,)
        self.args = a

    def launch(self, pdl: bool = False, stream=None):
        lib = _ext.require()
        self.heap.level_launch_counters(_ext.SITE_AGV_LL, self.grid)
        _ext.check(lib.mcb_launch_agv(C.byref(self.heap.ctx()), C.byref(self.args), self.grid, self.threads,
                                      int(pdl), _ext.stream_handle(stream)), "all_gather_v")


class ReduceScatterVPlan:
    """``out[t] = sum over ranks of src[offset + t]`` for this rank's rows; bf16 operands are
    accumulated in fp32 (in the switch with multimem), fp32 operands in fp32."""

    def __init__(self, heap: SymmetricHeap, out: torch.Tensor, src: HeapTensor, n_local, step_meta, cap: int,
                 site: int = _ext.SITE_RSV, grid: int = DEFAULT_GRID, threads: int = DEFAULT_THREADS,
                 ll_stage: HeapTensor | None = None, ll_rows: int = 0):
        _check_grid(grid, threads)
        rb = _row_bytes(out)
        _check_heap_tensor(heap, src, "reduce_scatter_v src")
        if out.dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("reduce_scatter_v supports bf16 and fp32")
        if out.dtype != src.tensor.dtype:
            raise ValueError("reduce_scatter_v: output and input dtypes differ")
        if rb % 16:
            raise ValueError(f"reduce_scatter_v rows must be multiples of 16 bytes (got {rb})")
        if out.shape[0] < cap or src.nbytes < cap * heap.world * rb:
            raise ValueError("reduce_scatter_v: buffers smaller than the capacity")
        self.heap, self.grid, self.threads = heap, grid, threads
        self._keep = (out, src, n_local, step_meta)
        a = _ext.McbRsvArgs()
        a.out, a.src_off, a.row_bytes = out.data_ptr(), src.offset, rb
        a.dtype = 1 if out.dtype == torch.float32 else 0
        a.cap, a.site = int(cap), int(site)
        a.n_local, a.step_meta = n_local.data_ptr(), step_meta.data_ptr()
        if ll_stage is not None and ll_rows > 0 and out.dtype == torch.bfloat16:
            need = rsv_ll_stage_bytes(heap.world, ll_rows, cap, rb)
            _check_heap_tensor(heap, ll_stage, "reduce_scatter_v low-latency staging")
            if ll_stage.nbytes < need:
                raise ValueError(f"low-latency staging holds {ll_stage.nbytes} bytes, {need} needed")
            a.ll_off, a.ll_rows, a.counts_off = ll_stage.offset, int(ll_rows), heap.counts_off
            a.ll_src_rows = min(int(cap), int(ll_rows))
            self._keep += (ll_stage,)
        self.args = a

    def launch(self, pdl: bool = False, stream=None):
        lib = _ext.require()
        self.heap.level_launch_counters(_ext.SITE_RSV_LL, self.grid)
        _ext.check(lib.mcb_launch_rsv(C.byref(self.heap.ctx()), C.byref(self.args), self.grid, self.threads,
                                      int(pdl), _ext.stream_handle(stream)), "reduce_scatter_v")


def dense_decode_step(heap, meta: MetadataPlan, agv: AllGatherVPlan, rsv: ReduceScatterVPlan,
                      num_layers: int, pdl: bool = False, stream=None):
    """metadata once, then ``num_layers`` x (all-gather-V, reduce-scatter-V), issued by one
    native call (bench_nvls.py:114-121 does this loop in Python)."""
    lib = _ext.require()
    heap.level_launch_counters(_ext.SITE_AGV_LL, agv.grid)
    heap.level_launch_counters(_ext.SITE_RSV_LL, agv.grid)
    _ext.check(lib.mcb_dense_decode_step(C.byref(heap.ctx()), C.byref(meta.args), C.byref(agv.args),
                                         C.byref(rsv.args), int(num_layers), agv.grid, agv.threads, int(pdl),
                                         _ext.stream_handle(stream)), "dense_decode_step")


def step_credit_bytes(grid: int = _ext.MAX_BLOCKS) -> int:
    """Heap bytes of the packet-mode credits of the step kernel: one word per (block, source rank)."""
    return int(grid) * _ext.MAX_RANKS * 4


class DenseStepPlan:
    """One whole decode step as ONE persistent kernel launch (``dense_step_kernel``): the count
    exchange, then ``num_layers`` x (push -> one cross-GPU barrier -> switch-side reduction), or
    packets without any barrier when the step holds at most ``ll_rows`` rows.

    ``dsts[i]`` are heap tensors of shape ``[2, cap * world, cols]``: the gathered rows are double
    buffered by layer parity (the barrier of a layer is then also the fence that protects the readers
    of the layer before).  After a step, ``step_meta[5]`` names the parity that holds the last layer's
    rows, ``step_meta[6]`` the mode (0 barrier, 1 packets) and ``step_meta[7]`` the number of
    pipeline groups used.  ``groups`` > 1 splits the blocks into groups that own a share of every
    rank's rows and take turns on the push, so that one group's reduction overlaps the next group's
    push (the two load opposite directions of the links); it needs ``grid`` <= number of SMs."""

    def __init__(self, heap: SymmetricHeap, dsts, srcs, out: torch.Tensor, rsv: HeapTensor, n_local, step_meta,
                 cap: int, num_layers: int, grid: int = DEFAULT_GRID, threads: int = DEFAULT_THREADS,
                 agv_ll_stage: HeapTensor | None = None, rsv_ll_stage: HeapTensor | None = None, ll_rows: int = 0,
                 groups: int = 1, group_min_bytes: int = 256 << 10, state: torch.Tensor | None = None,
                 credits: HeapTensor | None = None, check_errors: torch.Tensor | None = None, delay_ns: int = 0, delay_every: int = 1,
                 fp8_hidden: int = 0):
        """``fp8_hidden`` = H > 0 dispatches the hidden rows as 1 x 128 block-scaled e4m3: ``srcs[0]`` stays the
        bf16 ``[cap, H]`` input, ``dsts[0]`` is ``[2, cap * world, H]`` uint8, and a fourth pair
        ``(dsts[3], None)`` receives the fp32 scales ``[2, cap * world, H / 128]``."""
        if not (1 <= len(srcs) <= _ext.MAX_TENSORS) or len(srcs) != len(dsts):
            raise ValueError(f"need 1..{_ext.MAX_TENSORS} (dst, src) pairs")
        _check_grid(grid, threads)
        if not (1 <= groups <= _ext.MAX_GROUPS):
            raise ValueError(f"groups {groups} outside [1, {_ext.MAX_GROUPS}]")
        if groups > 1 and grid > DEFAULT_GRID:
            raise ValueError("pipeline groups wait on one another: the grid must not exceed the number of SMs")
        if step_meta.dtype != torch.int32 or step_meta.numel() < 8:
            raise ValueError("step_meta must be int32[8]")
        if n_local.dtype != torch.int32 or n_local.numel() != 1:
            raise ValueError("n_local must be an int32 scalar tensor on the device")
        if state is None:
            state = torch.zeros(_ext.STEP_STATE_WORDS, dtype=torch.int32, device=heap.device)
        if state.dtype != torch.int32 or state.numel() < _ext.STEP_STATE_WORDS:
            raise ValueError(f"state must be int32[{_ext.STEP_STATE_WORDS}]")
        self.heap, self.grid, self.threads, self.state = heap, grid, threads, state
        self._keep = (list(dsts), list(srcs), out, rsv, n_local, step_meta, agv_ll_stage, rsv_ll_stage)
        a = _ext.McbDenseStepArgs()
        gcap = cap * heap.world
        if fp8_hidden:
            if fp8_hidden % 128 or len(srcs) != 4 or srcs[3] is not None or check_errors is not None:
                raise ValueError("fp8 dispatch: hidden must be a multiple of 128 and the tensors "
                                 "(hidden, routing, probs, scales) with no source for the scales")
            if srcs[0].dtype != torch.bfloat16 or srcs[0].shape[1] != fp8_hidden or dsts[0].tensor.dtype != torch.uint8 \
                    or dsts[3].tensor.dtype != torch.float32 or dsts[3].tensor.shape[2] != fp8_hidden // 128:
                raise ValueError("fp8 dispatch: bf16 [cap, H] source, uint8 [2, rows, H] and fp32 [2, rows, H/128] gathered buffers")
        for i, (d, s) in enumerate(zip(dsts, srcs)):
            quant = bool(fp8_hidden) and i in (0, 3)
            rb = (fp8_hidden if i == 0 else fp8_hidden // 128 * 4) if quant else _row_bytes(s)
            _check_heap_tensor(heap, d, f"dense_step dst[{i}]")
            if rb % 4:
                raise ValueError(f"row of tensor {i} is {rb} bytes; must be a multiple of 4")
            if d.tensor.dim() != 3 or d.tensor.shape[0] != 2 or d.tensor.shape[1] < gcap:
                raise ValueError(f"tensor {i}: gathered buffer must be [2, >= cap * world, cols]")
            if not quant and (d.tensor.dtype != s.dtype or d.tensor.shape[2] != s.shape[1]):
                raise ValueError(f"tensor {i}: gathered buffer must have the source's dtype and columns")
            if s is not None:
                if s.shape[0] < cap:
                    raise ValueError(f"tensor {i}: source smaller than the capacity")
                if s.data_ptr() % 16:
                    raise ValueError(f"tensor {i}: source is not 16-byte aligned")
            a.src[i], a.dst_off[i], a.row_bytes[i] = (s.data_ptr() if s is not None else 0), d.offset, rb
            a.dst_par_stride[i] = d.tensor.shape[1] * rb
            if a.dst_par_stride[i] % 16:
                raise ValueError(f"tensor {i}: parity stride is not 16-byte aligned")
        rrb = _row_bytes(out)
        _check_heap_tensor(heap, rsv, "dense_step partial sums")
        if out.dtype not in (torch.bfloat16, torch.float32) or out.dtype != rsv.tensor.dtype:
            raise ValueError("combine supports bf16 and fp32, same dtype in and out")
        if rrb % 16 or out.shape[0] < cap or rsv.nbytes < gcap * rrb:
            raise ValueError("combine rows must be multiples of 16 bytes and buffers must hold the capacity")
        a.num_tensors, a.cap, a.num_layers = len(srcs), int(cap), int(num_layers)
        a.rsv_dtype = 1 if out.dtype == torch.float32 else 0
        a.out, a.rsv_off, a.rsv_row_bytes = out.data_ptr(), rsv.offset, rrb
        rbs = [int(a.row_bytes[i]) for i in range(len(srcs))]
        if ll_rows > 0 and agv_ll_stage is not None and rsv_ll_stage is not None and out.dtype == torch.bfloat16 \
                and all(rb % 8 == 0 for rb in rbs):
            need_a = agv_ll_stage_bytes(ll_rows, rbs)
            need_r = rsv_ll_stage_bytes(heap.world, ll_rows, cap, rrb)
            _check_heap_tensor(heap, agv_ll_stage, "dense_step packet staging (gather)")
            _check_heap_tensor(heap, rsv_ll_stage, "dense_step packet staging (reduce)")
            if agv_ll_stage.nbytes < need_a or rsv_ll_stage.nbytes < need_r:
                raise ValueError("packet staging areas are too small")
            if credits is None or credits.nbytes < step_credit_bytes(grid):
                raise ValueError(f"packet mode needs a zeroed heap region of {step_credit_bytes(grid)} bytes for its credits")
            _check_heap_tensor(heap, credits, "dense_step packet credits")
            a.ll_rows, a.ll_src_rows = int(ll_rows), min(int(cap), int(ll_rows))
            a.agv_ll_off, a.rsv_ll_off, a.credit_off = agv_ll_stage.offset, rsv_ll_stage.offset, credits.offset
            self._keep += (credits,)
        a.groups, a.group_min_bytes, a.fp8_hidden = int(groups), int(group_min_bytes), int(fp8_hidden)
        a.n_local, a.step_meta = n_local.data_ptr(), step_meta.data_ptr()
        a.counts_off, a.state = heap.step_counts_off, state.data_ptr()
        if check_errors is not None:
            # self-checking build: hashed payload verified by every receiver, optional per-layer sleep
            if check_errors.dtype != torch.int32 or check_errors.numel() < 1:
                raise ValueError("check_errors must be an int32 device counter")
            a.check_errors, a.check = check_errors.data_ptr(), 1
            a.delay_ns, a.delay_every = int(delay_ns), max(1, int(delay_every))
            self._keep += (check_errors,)
        self.args = a

    def launch(self, pdl: bool = False, stream=None):
        lib = _ext.require()
        _ext.check(lib.mcb_launch_dense_step(C.byref(self.heap.ctx()), C.byref(self.args), self.grid, self.threads,
                                             int(pdl), _ext.stream_handle(stream)), "dense_step")


# ---- uniform-count collectives (tensor-parallel style) ------------------------------------------
def _uniform_meta(heap: SymmetricHeap, rows_per_rank: int):
    dev = heap.device
    n_local = torch.tensor([rows_per_rank], dtype=torch.int32, device=dev)
    step_meta = torch.tensor([rows_per_rank * heap.world, rows_per_rank * heap.rank, rows_per_rank, 0],
                             dtype=torch.int32, device=dev)
    return n_local, step_meta


class UniformAllGatherPlan(AllGatherVPlan):
    """Equal-count all-gather of 1 to 4 tensors with one barrier (collectives.py:230-320 of the
    reference): rank r's rows land at ``[r * rows, (r + 1) * rows)``."""

    def __init__(self, heap, dsts, srcs, grid: int = DEFAULT_GRID, threads: int = DEFAULT_THREADS):
        rows = srcs[0].shape[0]
        if any(s.shape[0] != rows for s in srcs):
            raise ValueError("uniform all-gather: all sources need the same number of rows")
        n_local, step_meta = _uniform_meta(heap, rows)
        super().__init__(heap, dsts, srcs, n_local, step_meta, cap=rows, site=_ext.SITE_UNIFORM_AG,
                         grid=grid, threads=threads)


class UniformReduceScatterPlan(ReduceScatterVPlan):
    """Equal-count reduce-scatter (collectives.py:323-368): ``out`` = this rank's row block of
    the cross-rank sum."""

    def __init__(self, heap, out, src, grid: int = DEFAULT_GRID, threads: int = DEFAULT_THREADS):
        rows = out.shape[0]
        n_local, step_meta = _uniform_meta(heap, rows)
        super().__init__(heap, out, src, n_local, step_meta, cap=rows, site=_ext.SITE_UNIFORM_RS,
                         grid=grid, threads=threads)
