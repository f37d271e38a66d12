"""Single-GPU emulation of a multi-rank world.

All ranks of a collective run inside ONE cooperative kernel launch (grid.y = world), each
y-slice with its own context, heap, epochs and status words; "peer" pointers are simply the
other ranks' heaps on the same device.  This exercises the multi-rank protocol (offsets,
barriers, slot maps, counts) where only one GPU is available.  Separate launches per rank
would not do: kernels that wait on one another are never guaranteed to run concurrently.
Only the peer-access transport can be emulated (a multicast address needs real NVSwitch
members).
"""
from __future__ import annotations

import ctypes as C

import torch

from ..ops import _ext
from .symm_heap import (ALIGN, COUNTS_BYTES, FLAGS_BYTES, RESERVED_BYTES, STEP_COUNTS_BYTES, DeviceStatusError,
                        HeapTensor, _align)


def _to_device(structs, device) -> torch.Tensor:
    arr = (type(structs[0]) * len(structs))(*structs)
    return torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8).to(device)


class EmuWorld:
    def __init__(self, world: int, heap_bytes: int, device="cuda:0", timeout_s: float = 2.0,
                 phantom_ranks: int = 0):
        """``phantom_ranks`` extra ranks are counted in ``world`` but never run: barriers can then
        never complete, which is how the bounded-wait error path is exercised."""
        self.world, self.device = world, torch.device(device)
        self.total = world + phantom_ranks
        self.nbytes = _align(heap_bytes + RESERVED_BYTES, 4096)
        self.heaps = [torch.zeros(self.nbytes, dtype=torch.uint8, device=self.device) for _ in range(self.total)]
        self.epochs = [torch.zeros(_ext.NUM_SITES * _ext.MAX_BLOCKS, dtype=torch.int32, device=self.device)
                       for _ in range(world)]
        self.status = [torch.zeros(_ext.STATUS_WORDS, dtype=torch.int32, device=self.device) for _ in range(world)]
        self._cursor = RESERVED_BYTES
        self.ctxs = []
        for r in range(world):
            c = _ext.McbCtx()
            c.rank, c.world, c.transport = r, self.total, _ext.TRANSPORT_P2P
            c.timeout_ns = int(timeout_s * 1e9)
            c.heap_local, c.heap_mc, c.flags_off = self.heaps[r].data_ptr(), 0, 0
            c.epochs, c.status = self.epochs[r].data_ptr(), self.status[r].data_ptr()
            for p in range(self.total):
                c.heap_peer[p] = self.heaps[p].data_ptr()
            self.ctxs.append(c)
        self.d_ctx = _to_device(self.ctxs, self.device)
        self.counts_off = FLAGS_BYTES
        self._site_grid = {}
        self.step_counts_off = FLAGS_BYTES + COUNTS_BYTES
        self.a2a_counts_off = FLAGS_BYTES + COUNTS_BYTES + STEP_COUNTS_BYTES
        self.a2a_state = [torch.zeros(_ext.STEP_STATE_WORDS, dtype=torch.int32, device=self.device)
                          for _ in range(world)]
        self.step_state = [torch.zeros(_ext.STEP_STATE_WORDS, dtype=torch.int32, device=self.device)
                           for _ in range(world)]

    def alloc(self, shape, dtype) -> list[HeapTensor]:
        n = 1
        for s in shape:
            n *= int(s)
        esize = torch.empty((), dtype=dtype).element_size()
        off = self._cursor
        if off + n * esize > self.nbytes:
            raise MemoryError("emulated heap exhausted")
        self._cursor = _align(off + max(1, n * esize), ALIGN)
        return [HeapTensor(h[off:off + n * esize].view(dtype).view(*shape), off, n * esize) for h in self.heaps]

    def _level(self, site: int, grid: int):
        """Per-block launch counters need one grid per site: level the row when it changes
        (what SymmetricHeap.level_launch_counters does for a real rank)."""
        if self._site_grid.get(site) == grid:
            return
        if site in self._site_grid:
            for e in self.epochs:
                row = e[site * _ext.MAX_BLOCKS:(site + 1) * _ext.MAX_BLOCKS]
                row.fill_(int(row.max().item()))
        self._site_grid[site] = grid

    def upload(self, structs) -> torch.Tensor:
        return _to_device(structs, self.device)

    def check_status(self):
        for r in range(self.world):
            words = [int(v) & 0xFFFFFFFF for v in self.status[r].cpu().tolist()]
            if words[0]:
                raise DeviceStatusError(words)

    # ---- collectives over all emulated ranks -------------------------------------------------------
    def _stream(self):
        return _ext.stream_handle()

    def metadata(self, n_locals, step_metas, cap):
        args = []
        for r in range(self.world):
            a = _ext.McbMetaArgs()
            a.n_local, a.counts_off, a.step_meta, a.cap = n_locals[r].data_ptr(), self.counts_off, step_metas[r].data_ptr(), cap
            args.append(a)
        d = self.upload(args)
        _ext.check(_ext.require().mcb_emu_metadata(C.c_void_p(self.d_ctx.data_ptr()), C.c_void_p(d.data_ptr()),
                                                   self.world, self._stream()), "emu metadata")
        torch.cuda.synchronize()

    def all_gather_v(self, dsts, srcs, n_locals, step_metas, cap, grid=4, threads=256, site=_ext.SITE_AGV,
                     ll_stage=None, ll_rows=0):
        """dsts: list over tensors of per-rank HeapTensor lists; srcs: list over tensors of per-rank tensors."""
        args = []
        for r in range(self.world):
            a = _ext.McbAgvArgs()
            for i in range(len(srcs)):
                a.src[i], a.dst_off[i] = srcs[i][r].data_ptr(), dsts[i][r].offset
                a.row_bytes[i] = srcs[i][r].shape[1] * srcs[i][r].element_size()
            a.num_tensors, a.cap, a.site = len(srcs), cap, site
            a.n_local, a.step_meta = n_locals[r].data_ptr(), step_metas[r].data_ptr()
            if ll_stage is not None:
                a.ll_off, a.ll_rows = ll_stage[r].offset, ll_rows
            args.append(a)
        d = self.upload(args)
        self._level(_ext.SITE_AGV_LL, grid)
        _ext.check(_ext.require().mcb_emu_agv(C.c_void_p(self.d_ctx.data_ptr()), C.c_void_p(d.data_ptr()),
                                              self.world, grid, threads, self._stream()), "emu agv")
        torch.cuda.synchronize()

    def reduce_scatter_v(self, outs, src, n_locals, step_metas, cap, grid=4, threads=256, site=_ext.SITE_RSV,
                         ll_stage=None, ll_rows=0):
        args = []
        for r in range(self.world):
            a = _ext.McbRsvArgs()
            a.out, a.src_off = outs[r].data_ptr(), src[r].offset
            a.row_bytes = outs[r].shape[1] * outs[r].element_size()
            a.dtype = 1 if outs[r].dtype == torch.float32 else 0
            a.cap, a.site = cap, site
            a.n_local, a.step_meta = n_locals[r].data_ptr(), step_metas[r].data_ptr()
            if ll_stage is not None:
                a.ll_off, a.ll_rows, a.counts_off = ll_stage[r].offset, ll_rows, self.counts_off
                a.ll_src_rows = min(cap, ll_rows)
            args.append(a)
        d = self.upload(args)
        self._level(_ext.SITE_RSV_LL, grid)
        _ext.check(_ext.require().mcb_emu_rsv(C.c_void_p(self.d_ctx.data_ptr()), C.c_void_p(d.data_ptr()),
                                              self.world, grid, threads, self._stream()), "emu rsv")
        torch.cuda.synchronize()

    def dense_step(self, dsts, srcs, outs, rsv, n_locals, step_metas, cap, num_layers, grid=4, threads=256,
                   agv_ll_stage=None, rsv_ll_stage=None, ll_rows=0, groups=1, group_min_bytes=0,
                   check_errors=None, delays_ns=None, delay_every=1, fp8_hidden=0):
        """One persistent decode step on all emulated ranks.  dsts: list over tensors of per-rank
        HeapTensor lists of shape [2, cap * world, cols]; step_metas: per-rank int32[8]."""
        args = []
        for r in range(self.world):
            a = _ext.McbDenseStepArgs()
            for i in range(len(srcs)):
                if fp8_hidden and i in (0, 3):      # quantised rows / their scales (no source for the scales)
                    rb = fp8_hidden if i == 0 else fp8_hidden // 128 * 4
                else:
                    rb = srcs[i][r].shape[1] * srcs[i][r].element_size()
                a.src[i] = srcs[i][r].data_ptr() if srcs[i] is not None else 0
                a.dst_off[i], a.row_bytes[i] = dsts[i][r].offset, rb
                a.dst_par_stride[i] = dsts[i][r].tensor.shape[1] * rb
            a.num_tensors, a.cap, a.num_layers, a.fp8_hidden = len(srcs), cap, num_layers, fp8_hidden
            a.rsv_dtype = 1 if outs[r].dtype == torch.float32 else 0
            a.out, a.rsv_off = outs[r].data_ptr(), rsv[r].offset
            a.rsv_row_bytes = outs[r].shape[1] * outs[r].element_size()
            if agv_ll_stage is not None and ll_rows > 0:
                a.ll_rows, a.ll_src_rows = ll_rows, min(cap, ll_rows)
                a.agv_ll_off, a.rsv_ll_off = agv_ll_stage[r].offset, rsv_ll_stage[r].offset
                if getattr(self, "_step_credits", None) is None:
                    self._step_credits = self.alloc([_ext.MAX_BLOCKS * _ext.MAX_RANKS], torch.int32)
                a.credit_off = self._step_credits[r].offset
            a.groups, a.group_min_bytes = groups, group_min_bytes
            a.n_local, a.step_meta = n_locals[r].data_ptr(), step_metas[r].data_ptr()
            a.counts_off, a.state = self.step_counts_off, self.step_state[r].data_ptr()
            if check_errors is not None:
                a.check_errors, a.check = check_errors[r].data_ptr(), 1
                a.delay_ns, a.delay_every = (delays_ns[r] if delays_ns else 0), delay_every
            args.append(a)
        d = self.upload(args)
        _ext.check(_ext.require().mcb_emu_dense_step(C.c_void_p(self.d_ctx.data_ptr()), C.c_void_p(d.data_ptr()),
                                                     C.byref(args[0]), self.world, grid, threads, self._stream()),
                   "emu dense step")
        torch.cuda.synchronize()

    def moe_layer(self, ranks: list[dict], grid: int, topk: int, cap: int, ll_rows: int = 0, timeout_s: float = 2.0):
        """One whole MoE layer (``moe_layer_kernel``: dispatch, routing, experts, combine) on all
        emulated ranks in one cooperative launch; ``grid`` CTAs per rank, so grid * world must not
        exceed the number of SMs.  Each entry of ``ranks`` holds that rank's tensors: ``weights``
        (ExpertWeights), ``route`` (RouteBuffers), ``src`` = (hidden, routing, probs) local inputs,
        ``dst`` = (hidden, routing, probs) gathered HeapTensors, ``partial`` (HeapTensor), ``n_local``,
        ``step_meta``, ``act``, ``y``, ``out``, ``expert_begin`` and optionally ``ll_stage``."""
        stride = _ext.layer_args_size()
        blob = bytearray(stride * self.world)
        first = None
        for r, d in enumerate(ranks):
            p = _ext.McbLayerArgs()
            w, route = d["weights"], d["route"]
            C.memmove(C.addressof(p.ctx), C.addressof(self.ctxs[r]), C.sizeof(_ext.McbCtx))
            a = p.agv
            for i, (src, dst) in enumerate(zip(d["src"], d["dst"])):
                a.src[i], a.dst_off[i] = src.data_ptr(), dst.offset
                a.row_bytes[i] = src.shape[1] * src.element_size()
            a.num_tensors, a.cap, a.site = 3, cap, _ext.SITE_AGV
            a.n_local, a.step_meta = d["n_local"].data_ptr(), d["step_meta"].data_ptr()
            if ll_rows > 0:
                a.ll_off, a.ll_rows = d["ll_stage"].offset, ll_rows
            ro = p.route
            ro.topk_idx, ro.topk_w = d["dst"][1].tensor.data_ptr(), d["dst"][2].tensor.data_ptr()
            ro.num_tokens = d["step_meta"].data_ptr()
            ro.topk, ro.expert_begin, ro.num_local_experts, ro.max_tokens = topk, d["expert_begin"], route.E, route.max_tokens
            for f in ("expert_count", "expert_cursor", "expert_offset", "pair_token", "pair_prob", "pair_pos",
                      "tile_expert", "tile_row0", "tile_rows", "num_m_tiles", "sync", "max_rows", "ffn_done"):
                setattr(ro, f, getattr(route, f).data_ptr())
            ro.max_pairs, ro.max_tiles = route.max_pairs, route.max_tiles
            ro.status, ro.timeout_ns = self.status[r].data_ptr(), int(timeout_s * 1e9)
            ff = p.ffn
            ff.x, ff.x_row_bytes = d["dst"][0].tensor.data_ptr(), w.hidden * 2
            ff.pair_token, ff.pair_prob = route.pair_token.data_ptr(), route.pair_prob.data_ptr()
            ff.expert_offset, ff.max_rows = route.expert_offset.data_ptr(), route.max_rows.data_ptr()
            ff.act, ff.y, ff.ffn_done = d["act"].data_ptr(), d["y"].data_ptr(), route.ffn_done.data_ptr()
            ff.num_local_experts, ff.hidden, ff.intermediate = w.num_local_experts, w.hidden, w.intermediate
            ff.status, ff.timeout_ns = self.status[r].data_ptr(), int(timeout_s * 1e9)
            ff.w1, ff.w2 = w.w1.data_ptr(), w.w2.data_ptr()
            cm = p.cmb
            cm.y, cm.pair_pos, cm.partial_off, cm.out = d["y"].data_ptr(), route.pair_pos.data_ptr(), d["partial"].offset, d["out"].data_ptr()
            cm.n_local, cm.step_meta = d["n_local"].data_ptr(), d["step_meta"].data_ptr()
            cm.hidden, cm.topk, cm.cap, cm.site = w.hidden, topk, cap, _ext.SITE_FUSED_FC2
            if d["partial"].tensor.dim() == 3:
                cm.partial_par_stride = d["partial"].nbytes // 2
            blob[r * stride:r * stride + C.sizeof(p)] = bytes(p)
            if first is None:
                first = p
        dev_args = torch.frombuffer(blob, dtype=torch.uint8).to(self.device)
        if dev_args.data_ptr() % 64:
            raise RuntimeError("device allocation is not 64-byte aligned")
        _ext.check(_ext.require().mcb_emu_moe_layer(C.c_void_p(dev_args.data_ptr()), C.byref(first), self.world, grid,
                                                    self._stream()), "emu moe layer")
        torch.cuda.synchronize()

    def barrier_test(self, grid=2, rounds=1):
        _ext.check(_ext.require().mcb_emu_barrier_test(C.c_void_p(self.d_ctx.data_ptr()), self.world, grid, rounds,
                                                       self._stream()), "emu barrier test")
        torch.cuda.synchronize()

    def a2a_buffers(self, cap, hidden, topk, fp8):
        w = self.world
        b = {"cap": cap, "hidden": hidden, "topk": topk, "fp8": fp8}
        if fp8:
            b["recv_x"] = self.alloc([w, cap, hidden], torch.uint8)
            b["recv_scale"] = self.alloc([w, cap, hidden // 128], torch.float32)
            b["y"] = self.alloc([w, cap, hidden], torch.bfloat16)
        else:
            b["recv_x"] = self.alloc([w, cap, hidden], torch.bfloat16)
            b["recv_scale"] = None
            b["y"] = b["recv_x"]
        b["recv_idx"] = self.alloc([w, cap, topk], torch.int64)
        b["recv_w"] = self.alloc([w, cap, topk], torch.float32)
        b["recv_src"] = self.alloc([w, cap], torch.int32)
        b["recv_count"] = self.alloc([_ext.MAX_RANKS], torch.int32)
        b["slot_map"] = [torch.full((cap, w), -1, dtype=torch.int32, device=self.device) for _ in range(w)]
        b["send_count"] = [torch.zeros(_ext.MAX_RANKS + 1, dtype=torch.int32, device=self.device) for _ in range(w)]
        return b

    def a2a_dispatch(self, b, xs, idxs, ws, n_locals, num_experts, grid=4, threads=256):
        args = []
        for r in range(self.world):
            a = _ext.McbA2ADispatchArgs()
            a.x, a.topk_idx, a.topk_w = xs[r].data_ptr(), idxs[r].data_ptr(), ws[r].data_ptr()
            a.recv_x_off = b["recv_x"][r].offset
            a.recv_scale_off = b["recv_scale"][r].offset if b["recv_scale"] else 0
            a.recv_idx_off, a.recv_w_off = b["recv_idx"][r].offset, b["recv_w"][r].offset
            a.recv_src_off, a.recv_count_off = b["recv_src"][r].offset, b["recv_count"][r].offset
            a.slot_map, a.send_count = b["slot_map"][r].data_ptr(), b["send_count"][r].data_ptr()
            a.n_local = n_locals[r].data_ptr()
            a.hidden, a.topk, a.num_experts, a.cap, a.fp8 = b["hidden"], b["topk"], num_experts, b["cap"], int(b["fp8"])
            args.append(a)
        d = self.upload(args)
        _ext.check(_ext.require().mcb_emu_a2a_dispatch(C.c_void_p(self.d_ctx.data_ptr()), C.c_void_p(d.data_ptr()),
                                                       self.world, grid, threads, self._stream()), "emu a2a dispatch")
        torch.cuda.synchronize()

    def a2a_combine(self, b, outs, n_locals, grid=4, threads=256):
        args = []
        for r in range(self.world):
            a = _ext.McbA2ACombineArgs()
            a.out, a.y_off = outs[r].data_ptr(), b["y"][r].offset
            a.slot_map, a.n_local = b["slot_map"][r].data_ptr(), n_locals[r].data_ptr()
            a.hidden, a.cap = b["hidden"], b["cap"]
            args.append(a)
        d = self.upload(args)
        self._level(_ext.SITE_A2A_COMBINE, grid)
        _ext.check(_ext.require().mcb_emu_a2a_combine(C.c_void_p(self.d_ctx.data_ptr()), C.c_void_p(d.data_ptr()),
                                                      self.world, grid, threads, self._stream()), "emu a2a combine")
        torch.cuda.synchronize()

    def a2a_step_buffers(self, cap, hidden, topk, fp8, ll_rows=0):
        from ..ops.a2a import a2a_ll_specs, a2a_meta_row_bytes
        w = self.world
        b = {"cap": cap, "hidden": hidden, "topk": topk, "fp8": fp8, "meta_row_bytes": a2a_meta_row_bytes(topk),
             "ll_rows": ll_rows if w > 1 else 0}
        if b["ll_rows"] > 0:
            sx, sy, sc = a2a_ll_specs(w, cap, hidden, topk, fp8, ll_rows)
            b["ll_x"], b["ll_y"], b["credits"] = (self.alloc(sx[0], torch.uint8), self.alloc(sy[0], torch.uint8),
                                                  self.alloc(sc[0], torch.uint8))
            for t in b["credits"]:
                t.tensor.zero_()
        if fp8:
            b["recv_x"] = self.alloc([2, w, cap, hidden], torch.uint8)
            b["recv_scale"] = self.alloc([2, w, cap, hidden // 128], torch.float32)
            b["y"] = self.alloc([2, w, cap, hidden], torch.bfloat16)
        else:
            b["recv_x"] = self.alloc([2, w, cap, hidden], torch.bfloat16)
            b["recv_scale"] = None
            b["y"] = b["recv_x"]
        b["recv_meta"] = self.alloc([2, w, cap, b["meta_row_bytes"]], torch.uint8)
        return b

    def a2a_step(self, b, xs, idxs, ws, outs, n_locals, step_metas, num_experts, num_layers, grid=4, threads=256):
        """One persistent all-to-all decode step on all emulated ranks."""
        args = []
        for r in range(self.world):
            a = _ext.McbA2AStepArgs()
            a.x, a.topk_idx, a.topk_w, a.out = xs[r].data_ptr(), idxs[r].data_ptr(), ws[r].data_ptr(), outs[r].data_ptr()
            a.n_local = n_locals[r].data_ptr()
            a.recv_x_off, a.x_par_stride = b["recv_x"][r].offset, b["recv_x"][r].nbytes // 2
            if b["recv_scale"]:
                a.recv_scale_off, a.scale_par_stride = b["recv_scale"][r].offset, b["recv_scale"][r].nbytes // 2
            a.recv_meta_off, a.meta_par_stride = b["recv_meta"][r].offset, b["recv_meta"][r].nbytes // 2
            a.y_off, a.y_par_stride = b["y"][r].offset, b["y"][r].nbytes // 2
            a.meta_row_bytes, a.hidden, a.topk, a.num_experts = b["meta_row_bytes"], b["hidden"], b["topk"], num_experts
            a.cap, a.fp8, a.num_layers = b["cap"], int(b["fp8"]), num_layers
            a.step_meta, a.counts_off, a.state = step_metas[r].data_ptr(), self.a2a_counts_off, self.a2a_state[r].data_ptr()
            if b.get("ll_rows", 0) > 0:
                a.ll_rows, a.ll_src_rows = b["ll_rows"], min(b["cap"], b["ll_rows"])
                a.ll_x_off, a.ll_y_off, a.credit_off = b["ll_x"][r].offset, b["ll_y"][r].offset, b["credits"][r].offset
            args.append(a)
        d = self.upload(args)
        _ext.check(_ext.require().mcb_emu_a2a_step(C.c_void_p(self.d_ctx.data_ptr()), C.c_void_p(d.data_ptr()),
                                                   C.byref(self.ctxs[0]), C.byref(args[0]), self.world, grid, threads,
                                                   self._stream()), "emu a2a step")
        torch.cuda.synchronize()

    def rs_add_norm_ag(self, buf, residuals, weight, eps, grid=4):
        tokens, hidden = buf[0].tensor.shape
        args = []
        for r in range(self.world):
            a = _ext.McbNormArgs()
            a.buf_off, a.residual, a.weight = buf[r].offset, residuals[r].data_ptr(), weight.data_ptr()
            a.eps, a.hidden, a.tokens = eps, hidden, tokens
            args.append(a)
        d = self.upload(args)
        _ext.check(_ext.require().mcb_emu_rs_add_norm_ag(C.c_void_p(self.d_ctx.data_ptr()), C.c_void_p(d.data_ptr()),
                                                         self.world, hidden, grid, self._stream()), "emu norm")
        torch.cuda.synchronize()
