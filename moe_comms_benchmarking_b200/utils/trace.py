"""Host-side phase tracing: NVTX ranges (visible in Nsight tools) and, with ``MCB_TRACE=1``, a
wall-clock log of every phase on rank 0.  The reference has no instrumentation beyond one pair
of CUDA events (common.py:122-123, 161-172)."""
from __future__ import annotations

import contextlib
import os
import time

_LOG: list[tuple[str, float]] = []


def enabled() -> bool:
    return os.environ.get("MCB_TRACE", "0") not in ("", "0")


@contextlib.contextmanager
def phase(name: str, rank: int = 0):
    """``with phase("build"): ...`` opens an NVTX range when CUDA is present and records the
    host time of the block; with tracing enabled rank 0 prints it."""
    pushed = False
    try:
        import torch
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_push(name)
            pushed = True
    except Exception:
        pushed = False
    t0 = time.perf_counter()
    try:
        yield
    finally:
        dt = time.perf_counter() - t0
        _LOG.append((name, dt))
        if pushed:
            import torch
            torch.cuda.nvtx.range_pop()
        if enabled() and rank == 0:
            print(f"# [trace] {name}: {dt * 1e3:.2f} ms", flush=True)


def records() -> list[tuple[str, float]]:
    return list(_LOG)


def clear():
    _LOG.clear()
