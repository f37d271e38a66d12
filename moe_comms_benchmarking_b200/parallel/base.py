"""Dispatcher interface shared by every transport.

The reference's benchers are duck-typed (README.md:157, bench_*.py); here the protocol is a
small base class: ``build`` (collective allocation), ``setup_batch`` (load one step's
inputs), ``dispatch`` / ``combine`` / ``step`` / ``decode_step`` (the timed operations),
``validate`` (known-value checks -> ``[(name, ok, detail)]``), ``functional_roundtrip``
(dispatch -> identity expert -> combine on given tokens) and ``destroy``.
"""
from __future__ import annotations

import torch

from ..config import Config


class Dispatcher:
    name = "base"
    num_sms = -1          # CTA-count knob reported in the CSV (-1 = not applicable)

    def __init__(self, cfg: Config, group, device=None):
        self.cfg = cfg
        self.group = group
        if device is None:
            device = torch.device("cuda", cfg.local_rank) if torch.cuda.is_available() else torch.device("cpu")
        self.device = torch.device(device)
        self._built = False
        self.kernel_launches_per_step = lambda num_layers: 0

    # collective, once
    def build(self):
        raise NotImplementedError

    def setup_batch(self, hidden, topk_idx, topk_weights):
        raise NotImplementedError

    def dispatch(self):
        raise NotImplementedError

    def combine(self):
        raise NotImplementedError

    def step(self):
        self.dispatch()
        self.combine()

    def decode_step(self, num_layers: int):
        for _ in range(num_layers):
            self.step()

    def validate(self):
        return []

    def set_num_sms(self, num_sms: int):
        pass

    def check_health(self):
        """Raise if a kernel of this dispatcher reported an error (host-synchronising)."""

    def destroy(self):
        pass

    # helpers -----------------------------------------------------------------------------------
    def _validation_counts(self, global_b: int):
        w = self.cfg.ep_size
        return [global_b // w + (1 if r < global_b % w else 0) for r in range(w)]
