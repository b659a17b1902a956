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

__all__ = ["OffsetBasedRNGTracker", "is_rng_supported_mesh", "fork_rng", "local_shard_size_and_offset",
           "get_rng_tracker", "manual_seed", "distributed_rand_like"]


def is_rng_supported_mesh() -> bool:
    """Whether sharded random ops are supported here (reference random.py:31-45 asks the device
    handle for ``set_rng_state``).  Always true: CUDA generators expose their Philox state and the
    CPU generator is handled by re-seeding per offset window."""
    return True


def local_shard_size_and_offset(curr_local_size: int, num_chunks: int, rank: int):
    """``(size, start)`` of chunk ``rank`` when ``curr_local_size`` elements are split into
    ``num_chunks`` chunks the way ``torch.chunk`` does: chunks of ``ceil(size / chunks)``, a
    shorter last one, empty ones after it (their start is the end of the data).  Counterpart of
    reference random.py:386-419."""
    full = -(-curr_local_size // num_chunks)
    start = full * rank
    if start > curr_local_size:
        return 0, curr_local_size
    return min(curr_local_size, start + full) - start, start


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


# The three helpers below carry the names and argument lists of the reference's module-level
# functions (random.py:300-375 there); code that computes expected offsets with them keeps working.
def _calc_shard_info(mesh_coordinate, device_mesh, placements):
    """Per tensor dim: the index of this rank's shard and the number of shards, from the rank's mesh
    coordinate.  Several mesh dims sharding one tensor dim combine outer-to-inner.  Entries of
    ``placements`` that are not ``Shard`` count as replication."""
    from .placement_types import Shard
    mesh_shape = tuple(device_mesh.mesh_shape)
    by_dim = {}
    for i, p in enumerate(placements):
        if isinstance(p, Shard):
            by_dim.setdefault(p.dim, []).append(i)
    ndim = max([len(mesh_shape)] + [d + 1 for d in by_dim])
    idx, total = [0] * ndim, [1] * ndim
    for d, mesh_dims in by_dim.items():
        for m in mesh_dims:
            idx[d] = idx[d] * mesh_shape[m] + int(mesh_coordinate[m])
            total[d] *= mesh_shape[m]
    return idx, total


def _calc_shard_linear_idx(shard_coord, shard_size) -> int:
    """Row-major index of a shard coordinate."""
    lin = 0
    for c, n in zip(shard_coord, shard_size):
        lin = lin * int(n) + int(c)
    return lin


def _calc_first_shard_size(device_mesh, placements, global_shape):
    """Shape of the first (largest) shard: every sharded dim divided, rounding up, by the sizes of the
    mesh dims that shard it."""
    from .placement_types import Shard
    size = [int(g) for g in global_shape]
    for i, p in enumerate(placements):
        if isinstance(p, Shard) and p.dim < len(size):
            size[p.dim] = -(-size[p.dim] // int(device_mesh.mesh_shape[i]))
    return size


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

    _manual_seed = manual_seed          # the reference's spelling (random.py:119)

    @property
    def _device_handle(self):
        """The module that owns the generator the tracker drives (``torch.cuda`` or ``torch``)."""
        return torch.cuda if self.is_cuda else torch

    def _get_device_state(self) -> torch.Tensor:
        """The tracker's ``(seed, offset)`` as the 16 bytes of a Philox generator state, readable
        through :class:`_PhiloxState` on CPU too."""
        return torch.tensor([self._seed, self._offset], dtype=torch.int64).view(torch.uint8)

    def _set_pre_op_offset(self, state: _PhiloxState, device_mesh, placements, global_shape) -> None:
        """Advance ``state.offset`` to the window of this rank's shard (reference random.py:198-270)."""
        idx, total = _calc_shard_info(device_mesh.get_coordinate(), device_mesh, placements)
        numel = 1
        for n in _calc_first_shard_size(device_mesh, placements, global_shape):
            numel *= n
        state.offset = state.offset + _round4(_calc_shard_linear_idx(idx, total) * numel)

    def _set_post_op_offset(self, state: _PhiloxState, global_shape, old_offset: int) -> None:
        """Put ``state.offset`` past the whole tensor (reference random.py:272-292; a device mesh may be
        passed where the reference passes one: its shape is then what is counted, as there)."""
        shape = getattr(global_shape, "mesh_shape", global_shape)
        numel = 1
        for n in shape:
            numel *= int(n)
        state.offset = int(old_offset) + _round4(numel)

    @property
    def distribute_region_enabled(self) -> bool:
        """False: ``_distribute_region`` leaves offsets alone and random ops draw from the local generator."""
        return self._enabled

    @distribute_region_enabled.setter
    def distribute_region_enabled(self, value: bool) -> None:
        self._enabled = bool(value)

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
    def _distribute_region(self, layout=None, local_shape=None, global_shape: Optional[Sequence[int]] = None, *,
                           device_mesh=None, placements=None):
        """Random ops inside produce shard-consistent values for a tensor laid out as ``layout``.

        Two call forms: ``(layout, local_shape)``, and the reference's
        ``(device_mesh, placements, global_shape)`` (random.py:161-196), positional or by keyword.
        In the second form the window of a shard is sized by the first (largest) shard, so that
        every rank computes the same offsets when the tensor does not divide evenly.  The local
        generator state is restored on exit in both forms, also when the region is disabled."""
        if device_mesh is not None:
            layout, local_shape = device_mesh, placements
        if not isinstance(layout, Layout):
            from .dtensor import _build_layout
            if global_shape is None:
                raise TypeError("_distribute_region(device_mesh, placements, global_shape): global_shape is missing")
            global_shape = tuple(int(g) for g in global_shape)
            layout = _build_layout(layout, local_shape, len(global_shape))
            local_shape = list(global_shape)
            for d, axes in enumerate(layout.dim_axes):
                for a in axes:
                    local_shape[d] = -(-local_shape[d] // layout.mesh.mesh_shape[a])
        if not self._enabled:
            with self.fork_rng():
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


@contextlib.contextmanager
def fork_rng(devices=None, enabled: bool = True, device_type: str = "cuda"):
    """Save the CPU generator state and that of ``devices`` (default: every visible GPU) and put
    them back on exit; ``enabled=False`` does nothing.  Module-level counterpart of reference
    random.py:424-475."""
    if not enabled:
        yield
        return
    if devices is None:
        devices = range(torch.cuda.device_count()) if device_type == "cuda" and torch.cuda.is_available() else ()
    devices = list(devices)
    cpu_state = torch.get_rng_state()
    dev_states = [torch.cuda.get_rng_state(d) for d in devices]
    try:
        yield
    finally:
        torch.set_rng_state(cpu_state)
        for d, st in zip(devices, dev_states):
            torch.cuda.set_rng_state(st, d)


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
