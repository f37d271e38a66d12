"""CUDA-event / CUDA-graph timing with the reference's protocol (common.py:126-176):
eager warm-up, barrier, one side-stream warm-up and capture of ``fn`` as ONE graph,
``iters`` back-to-back replays between two events, per-iteration mean, max over ranks.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _events():
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def capture_graph(fn):
    """Warm ``fn`` on a side stream, then capture it into a ``torch.cuda.CUDAGraph``."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    torch.cuda.synchronize()
    return g


def time_region(fn, group, warmup: int, iters: int, use_graph: bool):
    """Returns ``(local_us, max_us)`` per iteration of ``fn``."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier(group)
    start, end = _events()
    if use_graph:
        g = capture_graph(fn)
        dist.barrier(group)
        start.record()
        for _ in range(iters):
            g.replay()
        end.record()
    else:
        start.record()
        for _ in range(iters):
            fn()
        end.record()
    torch.cuda.synchronize()
    local_us = start.elapsed_time(end) * 1e3 / iters
    t = torch.tensor([local_us], device=torch.cuda.current_device(), dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return local_us, float(t.item())


def timed_with_fallback(fn, group, warmup: int, iters: int, timing: str, rank: int = 0, log=print):
    """Graph timing that falls back to eager timing if capture fails (run.py:65-77).
    Returns ``((local_us, max_us), used_graph)``."""
    use_graph = timing == "graph"
    try:
        return time_region(fn, group, warmup, iters, use_graph), use_graph
    except Exception as e:
        if not use_graph:
            raise
        if rank == 0:
            log(f"  [warn] graph capture failed ({type(e).__name__}: {e}); falling back to eager", flush=True)
        dist.barrier(group)
        return time_region(fn, group, warmup, iters, False), False
