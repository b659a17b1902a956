"""Offline resharding between two layouts (hyper_parallel/core/checkpoint/reshard.py:88-398).

Pure index arithmetic on numpy / torch arrays: which slices of which source ranks make up the
slice that ``to_rank_id`` owns under ``to_layout``.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

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
    """Plans and performs the conversion of one parameter from ``from_layout`` to ``to_layout`` offline
    (numpy arrays or torch tensors, no process group).  Contract of the reference's class
    (core/checkpoint/reshard.py:190-398 there): ``infer_all_tensor_offset()`` names, per source rank
    that holds a needed and not redundant piece, the area of that piece *inside the source rank's
    shard*; the caller cuts those pieces out and hands them to ``get_real_tensor``, which places them
    into the target rank's shard.  A layout of ``None`` means the whole tensor on rank 0.  Beyond the
    reference, ``get_real_tensor`` also accepts the source ranks' whole shards and cuts the pieces
    itself."""

    def __init__(self, param_name: str, full_shape, from_layout: Optional[Layout], to_layout: Optional[Layout],
                 to_rank_id: int):
        if from_layout is None and to_layout is None:
            raise ValueError("`from_layout` and `to_layout` cannot both be None.")
        self.param_name = param_name
        self.full_shape = tuple(int(s) for s in full_shape)
        self.from_layout, self.to_layout = from_layout, to_layout

        def unpack(lay):
            if lay is None:
                return (1,), tuple(-1 for _ in self.full_shape), [0]
            if lay.tensor_map is None:
                lay.placement_to_tensor_map(len(self.full_shape))
            return tuple(lay.mesh_shape), tuple(lay.tensor_map), [int(r) for r in lay.rank_list]
        self.from_mesh_shape, self.from_tensor_map, self.from_rank_list = unpack(from_layout)
        self.to_mesh_shape, self.to_tensor_map, self.to_rank_list = unpack(to_layout)
        self.to_rank_id = 0 if to_layout is None else int(to_rank_id)
        if self.to_rank_id not in self.to_rank_list:
            raise ValueError("Input to_rank_id is not in to_rank_list.")
        self.to_area = infer_slice_area_by_rank(self.to_mesh_shape, self.to_tensor_map,
                                                self.to_rank_list.index(self.to_rank_id), self.full_shape)
        self.global_union_area_map: Dict[int, tuple] = {}     # source rank -> area of its piece in the full tensor
        self._from_area: Dict[int, tuple] = {}                 # source rank -> area of its whole shard

    def infer_all_tensor_offset(self) -> Dict[int, tuple]:
        """``{source rank: ((begin, end) per dim) inside that rank's shard}``: one entry per distinct
        source slice that overlaps the target shard (replicas are taken from the lowest rank)."""
        seen, out = set(), {}
        self.global_union_area_map.clear()
        self._from_area.clear()
        for inner, rank in enumerate(self.from_rank_list):
            src = tuple(infer_slice_area_by_rank(self.from_mesh_shape, self.from_tensor_map, inner, self.full_shape))
            if src in seen:
                continue
            seen.add(src)
            hit = infer_intersection(src, self.to_area)
            if hit is None:
                continue
            self.global_union_area_map[rank] = tuple(hit)
            self._from_area[rank] = src
            out[rank] = tuple((s - a0, e - a0) for (s, e), (a0, _) in zip(hit, src))
        return out

    def get_real_tensor(self, from_tensor_map: Dict[int, "np.ndarray"]):
        """The target rank's shard, assembled from ``{source rank: piece}`` (or ``{source rank: whole
        shard}``).  ``ValueError`` when a needed piece is missing or has neither of the two shapes."""
        if not from_tensor_map:
            raise ValueError("Input from_tensor_map cannot be empty")
        local = self.infer_all_tensor_offset()
        first = next(iter(from_tensor_map.values()))
        shape = [e - b for b, e in self.to_area]
        dst = first.new_zeros(shape) if hasattr(first, "new_zeros") else np.zeros(shape, dtype=first.dtype)
        for rank, area in self.global_union_area_map.items():
            if rank not in from_tensor_map:
                raise ValueError(f"{self.param_name}: missing slice data from rank {rank}; provide every slice that "
                                 "infer_all_tensor_offset names")
            piece = from_tensor_map[rank]
            want = tuple(e - b for b, e in area)
            whole = tuple(e - b for b, e in self._from_area[rank])
            if tuple(piece.shape) != want:
                if tuple(piece.shape) != whole:
                    raise ValueError(f"{self.param_name}: slice from rank {rank} has incorrect shape. Expected {want} "
                                     f"(or the whole shard {whole}), got {tuple(piece.shape)}.")
                piece = piece[tuple(slice(b, e) for b, e in local[rank])]
            dst[tuple(slice(b - t0, e - t0) for (b, e), (t0, _) in zip(area, self.to_area))] = piece
        return dst
