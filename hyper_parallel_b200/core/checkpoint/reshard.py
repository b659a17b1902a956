"""Offline resharding between two layouts (hyper_parallel/core/checkpoint/reshard.py:88-398).

Pure index arithmetic on numpy / torch arrays: which slices of which source ranks make up the
slice that ``to_rank_id`` owns under ``to_layout``.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import numpy as np

from ..layout import Layout, _infer_slice_area_by_rank


def infer_slice_area_by_rank(mesh_shape, tensor_map, rank_id: int, full_shape) -> List[Tuple[int, int]]:
    for axis, m in enumerate(tensor_map):
        ms = m if isinstance(m, (tuple, list)) else (m,)
        f = 1
        for a in ms:
            if a != -1:
                f *= mesh_shape[len(mesh_shape) - 1 - a]
        if full_shape[axis] % f:
            raise ValueError(f"dim {axis} of size {full_shape[axis]} is not divisible by {f}")
    return _infer_slice_area_by_rank(mesh_shape, tensor_map, rank_id, full_shape)


def infer_intersection(area_a, area_b):
    """Intersection of two ``[(begin, end)]`` boxes or ``None``."""
    out = []
    for (a0, a1), (b0, b1) in zip(area_a, area_b):
        s, e = max(a0, b0), min(a1, b1)
        if e <= s:
            return None
        out.append((s, e))
    return out


class ReshardHandler:
    """Plans and performs the conversion of one parameter from ``from_layout`` to ``to_layout``."""

    def __init__(self, param_name: str, full_shape, from_layout: Layout, to_layout: Layout, to_rank_id: int):
        self.param_name = param_name
        self.full_shape = tuple(full_shape)
        self.from_layout, self.to_layout = from_layout, to_layout
        self.to_rank_id = to_rank_id
        for lay in (from_layout, to_layout):
            if lay.tensor_map is None:
                lay.placement_to_tensor_map(len(self.full_shape))
        self.to_area = infer_slice_area_by_rank(to_layout.mesh_shape, to_layout.tensor_map,
                                                to_layout.rank_list.index(to_rank_id), self.full_shape)

    def infer_all_tensor_offset(self) -> Dict[int, Tuple[list, list]]:
        """``{source rank: (slice inside the source shard, slice inside the target shard)}`` --
        one entry per distinct source slice (replicas are taken from the lowest rank)."""
        seen, out = set(), {}
        for inner, rank in enumerate(self.from_layout.rank_list):
            src = infer_slice_area_by_rank(self.from_layout.mesh_shape, self.from_layout.tensor_map, inner,
                                           self.full_shape)
            key = tuple(src)
            if key in seen:
                continue
            hit = infer_intersection(src, self.to_area)
            if hit is None:
                continue
            seen.add(key)
            in_src = [(s - a0, e - a0) for (s, e), (a0, _) in zip(hit, src)]
            in_dst = [(s - b0, e - b0) for (s, e), (b0, _) in zip(hit, self.to_area)]
            out[rank] = (in_src, in_dst)
        return out

    def get_real_tensor(self, from_tensor_map: Dict[int, "np.ndarray"]):
        """Assemble the target shard from ``{source rank: source shard}``."""
        plan = self.infer_all_tensor_offset()
        first = next(iter(from_tensor_map.values()))
        shape = [e - b for b, e in self.to_area]
        is_torch = hasattr(first, "new_empty")
        dst = first.new_empty(shape) if is_torch else np.empty(shape, dtype=first.dtype)
        for rank, (in_src, in_dst) in plan.items():
            if rank not in from_tensor_map:
                raise KeyError(f"{self.param_name}: shard of source rank {rank} is required but missing")
            s = tuple(slice(b, e) for b, e in in_src)
            d = tuple(slice(b, e) for b, e in in_dst)
            dst[d] = from_tensor_map[rank][s]
        return dst
