"""Host-side capability checks, asked before anything is launched (a shared GPU is never
probed by faulting it).

Counterparts of ``is_device_nvls_capable`` / ``are_tensors_nvls_eligible``
(nvls/torch_symm_triton/utils.py:20-39), extended by what this library can actually tell:
whether the heap really has a multicast address, and which access width a row allows.
"""
from __future__ import annotations

import torch


def is_device_multimem_capable(device) -> bool:
    """``multimem.*`` instructions need a CUDA device of compute capability 9.0 or newer (and, at
    run time, an NVSwitch multicast object: see ``heap_has_multicast``)."""
    device = torch.device(device)
    if device.type != "cuda" or not torch.cuda.is_available():
        return False
    return torch.cuda.get_device_properties(device).major >= 9


def is_device_tcgen05_capable(device) -> bool:
    """The grouped GEMMs are built for sm_100a only (tcgen05, TMEM)."""
    device = torch.device(device)
    if device.type != "cuda" or not torch.cuda.is_available():
        return False
    return torch.cuda.get_device_properties(device).major == 10


def heap_has_multicast(heap) -> bool:
    """True when the symmetric heap was bound to a multicast object (world > 1, NVLS present)."""
    return bool(getattr(heap, "mc_ptr", 0))


def row_access_bytes(t: torch.Tensor) -> int:
    """Widest access the collectives use for rows of ``t``: 16, 8 or 4 bytes; 0 if ``t`` cannot
    be sent (not 2-D / not contiguous / row not a multiple of 4 bytes)."""
    if t.dim() != 2 or not t.is_contiguous():
        return 0
    rb = t.shape[1] * t.element_size()
    for width in (16, 8, 4):
        if rb % width == 0:
            return width
    return 0


def are_tensors_gather_eligible(*tensors: torch.Tensor) -> bool:
    """All-gather-V accepts 2-D contiguous tensors whose rows are multiples of 4 bytes."""
    return bool(tensors) and all(row_access_bytes(t) > 0 for t in tensors)


def are_tensors_reduce_eligible(*tensors: torch.Tensor) -> bool:
    """Reduce-scatter-V accepts bf16 or fp32 2-D contiguous tensors with rows of 16-byte multiples
    (the reference's rule: byte size divisible by 16)."""
    return bool(tensors) and all(t.dtype in (torch.bfloat16, torch.float32) and row_access_bytes(t) == 16
                                 for t in tensors)
