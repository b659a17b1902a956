"""Distributed random numbers for sharded tensors.

Capability of hyper_parallel/core/random.py:48-475 of the reference (itself modelled on torch
DTensor's ``OffsetBasedRNGTracker``): all ranks share one Philox ``(seed, offset)``; inside
``_distribute_region(layout, local_shape)`` each *distinct shard* draws from its own offset
window ``shard_linear_index * local_numel`` (rounded up to a multiple of 4), replicas of a shard
draw identical numbers, and afterwards every rank advances the offset by the global numel so
that the next op starts from the same point everywhere.

CUDA generators expose the Philox state directly (16 bytes: seed, offset).  On CPU (Mersenne
Twister, no offsets) the tracker emulates the windows by re-seeding with ``hash(seed, offset)``,
which keeps the same guarantees (shard-distinct, replica-identical, rank-consistent sequence).
"""
from __future__ import annotations

import contextlib
import logging
from typing import Optional, Sequence

import torch

from ..collectives import cc
from .layout import Layout

logger = logging.getLogger(__name__)


class _PhiloxState:
    """View of a CUDA generator state as (seed, offset)."""

    def __init__(self, state: torch.Tensor):
        self.state = state.clone()

    @property
    def seed(self) -> int:
        return int(self.state[:8].view(torch.int64).item())

    @seed.setter
    def seed(self, v: int) -> None:
        self.state[:8] = torch.tensor([v], dtype=torch.int64).view(torch.uint8)

    @property
    def offset(self) -> int:
        return int(self.state[8:16].view(torch.int64).item())

    @offset.setter
    def offset(self, v: int) -> None:
        self.state[8:16] = torch.tensor([v], dtype=torch.int64).view(torch.uint8)


def _round4(n: int) -> int:
    return (n + 3) // 4 * 4


class OffsetBasedRNGTracker:
    def __init__(self, device: Optional[torch.device] = None, run_state_sync: bool = True, seed: int = 0):
        self.device = torch.device(device) if device is not None else (
            torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        self.is_cuda = self.device.type == "cuda"
        self._seed = seed
        self._offset = 0
        self._enabled = True
        if self.is_cuda:
            st = _PhiloxState(torch.cuda.get_rng_state(self.device))
            self._seed, self._offset = st.seed, st.offset
        if run_state_sync:
            self.sync_state()

    # ------------------------------------------------------------------ sync --
    def sync_state(self, src: int = 0, group=None) -> None:
        """Broadcast rank ``src``'s (seed, offset) so every rank starts from the same state."""
        if not cc.is_initialized():
            return
        t = torch.tensor([self._seed, self._offset], dtype=torch.int64,
                         device=self.device if (self.is_cuda and cc.get_backend() == "nccl") else "cpu")
        cc.broadcast(t, src=src, group=group)
        self._seed, self._offset = int(t[0].item()), int(t[1].item())

    def manual_seed(self, seed: int) -> None:
        self._seed, self._offset = int(seed), 0

    def get_seed(self) -> int:
        return self._seed

    def get_offset(self) -> int:
        return self._offset

    def set_offset(self, offset: int) -> None:
        self._offset = int(offset)

    # ----------------------------------------------------------------- region --
    @staticmethod
    def shard_linear_index(layout: Layout, rank: Optional[int] = None) -> int:
        """Row-major index of this rank's shard among the distinct shards of the tensor."""
        mesh = layout.mesh
        coord = mesh.get_coordinate() if rank is None else mesh.coordinate_of(rank)
        idx = 0
        for axes in layout.dim_axes:
            for a in axes:
                idx = idx * mesh.mesh_shape[a] + coord[a]
        return idx

    @contextlib.contextmanager
    def _distribute_region(self, layout: Layout, local_shape: Sequence[int]):
        """Random ops inside produce shard-consistent values for a tensor laid out as ``layout``."""
        if not self._enabled:
            yield
            return
        local_numel = 1
        for s in local_shape:
            local_numel *= int(s)
        n_shards = 1
        for axes in layout.dim_axes:
            for a in axes:
                n_shards *= layout.mesh.mesh_shape[a]
        start = self._offset + _round4(self.shard_linear_index(layout) * local_numel)
        with self.fork_rng():
            self._set_device_state(self._seed, start)
            yield
        self._offset = self._offset + _round4(n_shards * local_numel)

    def _set_device_state(self, seed: int, offset: int) -> None:
        if self.is_cuda:
            st = _PhiloxState(torch.cuda.get_rng_state(self.device))
            st.seed, st.offset = seed, offset
            torch.cuda.set_rng_state(st.state, self.device)
        else:
            torch.manual_seed((seed * 1000003 + offset * 7919) % (2 ** 63 - 1))

    @contextlib.contextmanager
    def fork_rng(self):
        """Save the device generator state and restore it on exit."""
        if self.is_cuda:
            saved = torch.cuda.get_rng_state(self.device)
            try:
                yield
            finally:
                torch.cuda.set_rng_state(saved, self.device)
        else:
            saved = torch.get_rng_state()
            try:
                yield
            finally:
                torch.set_rng_state(saved)

    @contextlib.contextmanager
    def disabled(self):
        prev, self._enabled = self._enabled, False
        try:
            yield
        finally:
            self._enabled = prev


_TRACKER: Optional[OffsetBasedRNGTracker] = None


def get_rng_tracker() -> OffsetBasedRNGTracker:
    global _TRACKER
    if _TRACKER is None:
        _TRACKER = OffsetBasedRNGTracker()
    return _TRACKER


def manual_seed(seed: int) -> None:
    """Seed the distributed tracker (call with the same value on every rank)."""
    get_rng_tracker().manual_seed(seed)


def distributed_rand_like(fn, size, layout: Layout, **kwargs) -> torch.Tensor:
    """Draw this rank's shard of a random tensor of global ``size`` laid out as ``layout``."""
    local_shape = layout.get_local_shape(size)
    with get_rng_tracker()._distribute_region(layout, local_shape):
        return fn(local_shape, **kwargs)
