"""Host-side membership and health checks.

The reference has no failure detection of its own: its cross-GPU barrier spins forever if a
peer never arrives (nvls/torch_symm_triton/barrier.py:28-31,50-53), and the only timeouts
belong to the external DeepEP buffer (bench_deepep.py:49-50).  Here a failure is caught at
two levels: on the device every wait is bounded and reports through the status words
(``SymmetricHeap.check_status``); on the host ranks publish their state in the process
group's key-value store, so the others learn that a rank left *before* their next launch
instead of waiting inside a kernel for a peer that is gone.
"""
from __future__ import annotations

import time

import torch.distributed as dist


class RankLeft(RuntimeError):
    def __init__(self, ranks):
        super().__init__(f"rank(s) {sorted(ranks)} left the job")
        self.ranks = sorted(ranks)


class Membership:
    """``beat(step)`` records progress, ``leave()`` announces a clean departure (call it only
    between steps, with no kernel or collective in flight), ``check()`` raises ``RankLeft`` if
    any rank has left, ``stale(seconds)`` lists ranks whose heartbeat is older than that."""

    def __init__(self, rank: int, world: int, store=None, prefix: str = "mcb/member"):
        self.rank, self.world, self.prefix = rank, world, prefix
        self.store = store if store is not None else dist.distributed_c10d._get_default_store()
        self.store.set(f"{prefix}/{rank}/state", "alive")
        self.beat(0)

    def beat(self, step: int):
        self.store.set(f"{self.prefix}/{self.rank}/beat", f"{step}:{time.time():.3f}")

    def leave(self):
        self.store.set(f"{self.prefix}/{self.rank}/state", "left")

    def _get(self, key: str):
        try:
            if hasattr(self.store, "check") and not self.store.check([key]):
                return None
            return self.store.get(key).decode()
        except Exception:
            return None

    def left(self) -> list[int]:
        return [r for r in range(self.world) if self._get(f"{self.prefix}/{r}/state") == "left"]

    def check(self):
        gone = self.left()
        if gone:
            raise RankLeft(gone)

    def stale(self, seconds: float) -> list[int]:
        now, out = time.time(), []
        for r in range(self.world):
            v = self._get(f"{self.prefix}/{r}/beat")
            if v is None or now - float(v.split(":")[1]) > seconds:
                out.append(r)
        return out
