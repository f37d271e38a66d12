"""Decode engine: the user-facing object that owns a dispatcher, captures one decode step
(``num_layers`` MoE layers) as a CUDA graph once, and replays it for every step.

This is the framework's public entry point for serving-style use; the reference only has
the benchmark loop (run.py:200-226) and re-captures a graph per batch size, because its
kernels bake the local token count into the launch.  Here the count is a device scalar, so
the graph captured at the capacity serves any batch.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..config import Config
from ..utils.timing import capture_graph


class MoEDecodeEngine:
    def __init__(self, cfg: Config, group, impl: str = "dense", num_layers: int = 88, use_graph: bool = True,
                 **dispatcher_kwargs):
        self.cfg, self.group, self.num_layers, self.use_graph = cfg, group, num_layers, use_graph
        if impl == "dense":
            from ..parallel.dense import DenseDispatcher
            self.dispatcher = DenseDispatcher(cfg, group, **dispatcher_kwargs)
        elif impl == "a2a":
            from ..parallel.a2a import A2ADispatcher
            self.dispatcher = A2ADispatcher(cfg, group, **dispatcher_kwargs)
        elif impl == "nccl":
            from ..parallel.nccl import NCCLDispatcher
            self.dispatcher = NCCLDispatcher(cfg, group)
        elif impl == "fused":
            from ..parallel.fused import FusedExpertDispatcher
            self.dispatcher = FusedExpertDispatcher(cfg, group, **dispatcher_kwargs)
        else:
            raise ValueError(f"unknown impl {impl!r}")
        self.impl = impl
        self.graph = None
        self._pinned = None

    def build(self):
        self.dispatcher.build()
        return self

    def capture(self):
        """Capture the decode step once.  Collective: every rank captures the same graph."""
        d = self.dispatcher
        if self.impl == "nccl":
            raise RuntimeError("the NCCL baseline pads to a per-batch count and is captured per batch by the "
                               "benchmark driver; the engine serves the native dispatchers")
        d.decode_step(self.num_layers)       # warm-up outside capture
        torch.cuda.synchronize()
        dist.barrier(self.group)
        if self.use_graph:
            self.graph = capture_graph(lambda: d.decode_step(self.num_layers))
        dist.barrier(self.group)
        return self

    def load_batch(self, hidden, topk_idx, topk_weights):
        """Device tensors of this rank's tokens for the next step."""
        self.dispatcher.setup_batch(hidden, topk_idx, topk_weights)

    def run(self):
        """Replay the captured step (or issue it eagerly)."""
        if self.graph is not None:
            self.graph.replay()
        else:
            self.dispatcher.decode_step(self.num_layers)

    def step_host(self, hidden_pinned, idx_pinned, w_pinned, out_pinned=None):
        """End-to-end step from pinned host tensors: H2D of the inputs, the decode step, D2H of
        the combined output of the last layer.  Returns the pinned output ``[n, H]`` (valid after
        this call returns: it synchronises)."""
        d = self.dispatcher
        n = hidden_pinned.shape[0]
        if n > d.cap:
            raise ValueError(f"{n} tokens exceed the per-rank capacity {d.cap}")
        if self._pinned is None:
            self._pinned = {"n": torch.zeros(1, dtype=torch.int32).pin_memory(),
                            "out": torch.empty(d.cap, self.cfg.hidden, dtype=d.out_buf.dtype).pin_memory()}
        self._pinned["n"][0] = n
        if n:
            d.in_hidden[:n].copy_(hidden_pinned, non_blocking=True)
            d.in_routing[:n].copy_(idx_pinned, non_blocking=True)
            d.in_probs[:n].copy_(w_pinned, non_blocking=True)
        d.n_local.copy_(self._pinned["n"], non_blocking=True)
        d.local_tokens = n
        self.run()
        out = out_pinned if out_pinned is not None else self._pinned["out"]
        if n:
            out[:n].copy_(d.out_buf[:n], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return out[:n]

    def check_health(self):
        self.dispatcher.check_health()

    def destroy(self):
        self.graph = None
        self.dispatcher.destroy()
