"""Host-side failure detection: heartbeats through the rendezvous store, and kernel status words.

The reference has none (only ``timeout`` arguments forwarded to process-group creation).  Two
mechanisms are provided:

* every fused kernel records a code in a per-device status word when a bounded wait expires;
  ``check_kernel_status()`` turns that into an exception after a step;
* ``Heartbeat`` publishes a per-rank counter in the ``torch.distributed`` store; ``dead_ranks()``
  lists ranks whose counter has not moved for ``timeout`` seconds, so that the survivors can stop
  launching collectives (and reload a checkpoint on fewer ranks) instead of hanging in one.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional

import torch.distributed as dist

from ..ops import native


def check_kernel_status(device=None) -> None:
    native.check_status(device)


class Heartbeat:
    def __init__(self, store=None, rank: Optional[int] = None, world_size: Optional[int] = None,
                 prefix: str = "hpb_heartbeat"):
        if store is None:
            store = dist.distributed_c10d._get_default_store()
        self.store = store
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world_size is None else world_size
        self.prefix = prefix
        self.count = 0
        self.store_lost = False
        self._seen: Dict[int, tuple] = {}

    def beat(self) -> None:
        """Publish this rank's counter.  If the store cannot be reached (the rank that hosts it has
        gone) the error is kept in ``store_lost`` instead of being raised: ``dead_ranks`` then sees no
        counter move and reports the others, the store's host among them, after its timeout."""
        self.count += 1
        try:
            self.store.set(f"{self.prefix}/{self.rank}", str(self.count))
        except Exception:  # noqa: BLE001 - DistNetworkError / RuntimeError, depending on the store
            self.store_lost = True

    def _read(self, r: int) -> int:
        try:
            if not self.store.check([f"{self.prefix}/{r}"]):
                return -1
            return int(self.store.get(f"{self.prefix}/{r}"))
        except Exception:  # noqa: BLE001 - a store error is treated as "no progress"
            return -1

    def dead_ranks(self, timeout: float) -> List[int]:
        """Ranks whose heartbeat did not advance during the last ``timeout`` seconds."""
        now = time.monotonic()
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            v = self._read(r)
            last = self._seen.get(r)
            if last is None or v != last[0]:
                self._seen[r] = (v, now)
            elif now - last[1] > timeout:
                dead.append(r)
        return dead
