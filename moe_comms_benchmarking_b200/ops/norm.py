"""Fused reduce-scatter + residual add + RMSNorm + all-gather (tensor-parallel decode op).

Counterpart of ``fused_multimem_rs_add_norm_ag`` (nvls/torch_symm_triton/fused_collectives.py:210-280).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _ext
from .dense import _check_heap_tensor
from ..parallel.symm_heap import HeapTensor, SymmetricHeap


class RsAddNormAgPlan:
    """In place on ``buf`` (heap, bf16 ``[tokens, hidden]``): every rank's ``buf`` holds partial
    sums going in and the normalised rows of all tokens coming out; ``residual``
    (``[tokens / world, hidden]`` bf16, local) is updated to ``sum + residual``."""

    def __init__(self, heap: SymmetricHeap, buf: HeapTensor, residual: torch.Tensor, weight: torch.Tensor,
                 eps: float = 1e-5, grid: int = 128):
        t = buf.tensor
        if t.dtype != torch.bfloat16 or t.dim() != 2:
            raise ValueError("buf must be a bf16 [tokens, hidden] heap tensor")
        tokens, hidden = t.shape
        if tokens % heap.world:
            raise ValueError("tokens must be divisible by the world size")
        if hidden % 8 or hidden > 8192:
            raise ValueError("hidden must be a multiple of 8 and at most 8192")
        if residual.dtype != torch.bfloat16 or tuple(residual.shape) != (tokens // heap.world, hidden) \
                or not residual.is_contiguous():
            raise ValueError("residual must be contiguous bf16 [tokens/world, hidden]")
        if weight.dtype != torch.bfloat16 or weight.numel() != hidden:
            raise ValueError("weight must be bf16 [hidden]")
        if not (1 <= grid <= _ext.MAX_BLOCKS):
            raise ValueError("grid out of range")
        _check_heap_tensor(heap, buf, "rs_add_norm_ag buf")
        self.heap, self.grid = heap, grid
        self._keep = (buf, residual, weight)
        a = _ext.McbNormArgs()
        a.buf_off, a.residual, a.weight = buf.offset, residual.data_ptr(), weight.data_ptr()
        a.eps, a.hidden, a.tokens = float(eps), hidden, tokens
        self.args = a

    def launch(self, pdl: bool = False, stream=None):
        lib = _ext.require()
        _ext.check(lib.mcb_launch_rs_add_norm_ag(C.byref(self.heap.ctx()), C.byref(self.args), self.grid,
                                                 int(pdl), _ext.stream_handle(stream)), "rs_add_norm_ag")
