"""Shape helpers (hyper_parallel/core/utils.py:15-32 of the reference)."""
from __future__ import annotations

from typing import Sequence, Tuple

from .device_mesh import DeviceMesh
from .dtensor import _build_layout, compute_local_shape_and_offset
from .placement_types import Placement


def compute_local_shape_and_global_offset(global_shape: Sequence[int], device_mesh: DeviceMesh,
                                          placements: Sequence[Placement]) -> Tuple[tuple, tuple]:
    """Local shard shape and its offset inside the global tensor for this rank (``torch.chunk``
    semantics where a dimension does not divide evenly)."""
    layout = _build_layout(device_mesh, tuple(placements), len(global_shape))
    return compute_local_shape_and_offset(global_shape, layout)
