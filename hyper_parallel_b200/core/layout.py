"""``Layout``: how a tensor is laid out over a :class:`DeviceMesh`.

Behaviour follows hyper_parallel/core/layout.py:99-617 of the reference: a layout
is created from a mesh shape + axis aliases, and *calling* it with one entry per
tensor dimension (axis aliases, tuples of aliases, ``"None"``) or with one
placement per mesh dimension returns a configured copy.

Internally a layout is ``dim_axes`` -- for every tensor dim the tuple of mesh-dim
indices that shard it, outermost split first -- plus one pending-reduction tag
per mesh dim.  The reference's views are derived from that:

* ``tensor_map``: per tensor dim ``-1`` (not sharded), or the **reversed** mesh
  index ``ndim-1-i``, or a tuple of those for multi-axis sharding;
* ``alias_tensor_map``: the same with axis names / ``"None"``;
* ``placements``: one ``Shard/Replicate/Partial`` per mesh dim;
* ``partial``: per mesh dim ``None`` or one of ``sum max min avg prod all``.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple, Union

import numpy as np

from .device_mesh import DeviceMesh, _create_device_mesh
from .placement_types import Partial, Placement, Replicate, Shard

_PARTIAL_OPS = ("sum", "max", "min", "avg", "prod", "all")
DimAxes = Tuple[Tuple[int, ...], ...]


def _coord_of_inner_rank(mesh_shape: Sequence[int], inner_rank: int) -> List[int]:
    coord = [0] * len(mesh_shape)
    for i in range(len(mesh_shape) - 1, -1, -1):
        coord[i] = inner_rank % mesh_shape[i]
        inner_rank //= mesh_shape[i]
    return coord


def _infer_slice_area_by_rank(mesh_shape, tensor_map, rank_id: int, full_shape) -> List[Tuple[int, int]]:
    """``[(begin, end)]`` per tensor dim of the slice that inner rank ``rank_id`` owns.

    ``tensor_map`` uses the reversed-index convention; in a tuple the first axis is
    the outer split.
    """
    nd = len(mesh_shape)
    coord = _coord_of_inner_rank(mesh_shape, rank_id)
    area = []
    for axis, full in enumerate(full_shape):
        m = tensor_map[axis]
        ms = m if isinstance(m, (tuple, list)) else (m,)
        split, idx = 1, 0
        for a in ms:
            if a == -1:
                continue
            size = mesh_shape[nd - 1 - a]
            idx = idx * size + coord[nd - 1 - a]
            split *= size
        if full % split:
            raise ValueError(f"dim {axis} of size {full} is not divisible by {split}")
        step = full // split
        area.append((idx * step, (idx + 1) * step))
    return area


def _get_slice_tensor_by_layout(global_tensor, layout: "Layout"):
    """This rank's slice (a copy) of a replicated global tensor."""
    inner = layout.rank_list.index(layout.mesh.rank)
    area = _infer_slice_area_by_rank(layout.mesh_shape, layout.tensor_map, inner, global_tensor.shape)
    return global_tensor[tuple(slice(b, e) for b, e in area)].clone()


def _infer_slice_shape_by_layout(global_shape, layout: "Layout") -> List[int]:
    out = []
    for n, axes in zip(global_shape, layout.dim_axes):
        f = 1
        for a in axes:
            f *= layout.mesh_shape[a]
        out.append(int(n) // f)
    return out


class Layout:
    """Distribution of a tensor over a device mesh (see module docstring)."""

    def __init__(self, mesh_shape, alias_name, rank_list=None, init_backend=True):
        mesh_shape = tuple(int(s) for s in mesh_shape)
        alias_name = tuple(alias_name)
        if len(mesh_shape) != len(alias_name):
            raise ValueError(f"mesh_shape {mesh_shape} and alias_name {alias_name} differ in length")
        if rank_list is None or len(rank_list) == 0:
            rank_list = tuple(range(int(np.prod(mesh_shape))))
        mesh = _create_device_mesh("cuda", mesh_shape, mesh_dim_names=alias_name,
                                   rank_list=tuple(rank_list), init_backend=init_backend)
        self._setup(mesh)

    def _setup(self, mesh: DeviceMesh):
        self._mesh = mesh
        self._dim_axes: Optional[DimAxes] = None
        self._partial: List[Optional[str]] = [None] * mesh.ndim
        self._pending_placements: Optional[Tuple[Placement, ...]] = None
        self._compact: Optional[str] = None

    @classmethod
    def from_device_mesh(cls, device_mesh: DeviceMesh) -> "Layout":
        obj = cls.__new__(cls)
        obj._setup(device_mesh)
        return obj

    @classmethod
    def _make(cls, mesh: DeviceMesh, dim_axes: Sequence[Sequence[int]],
              partial: Optional[Sequence[Optional[str]]] = None) -> "Layout":
        """Fast constructor used by the op rules."""
        obj = cls.__new__(cls)
        obj._mesh = mesh
        obj._dim_axes = tuple(tuple(a) for a in dim_axes)
        obj._partial = list(partial) if partial is not None else [None] * mesh.ndim
        obj._pending_placements = None
        obj._compact = None
        return obj

    def copy(self) -> "Layout":
        obj = Layout.__new__(Layout)
        obj._mesh = self._mesh
        obj._dim_axes = self._dim_axes
        obj._partial = list(self._partial)
        obj._pending_placements = self._pending_placements
        obj._compact = self._compact
        return obj

    __copy__ = copy

    def __deepcopy__(self, memo):
        return self.copy()

    # ---------------------------------------------------------- calling ---
    def __call__(self, *spec) -> "Layout":
        if len(spec) == 1 and isinstance(spec[0], (list, tuple)) and len(spec[0]) > 0 \
                and isinstance(spec[0][0], Placement):
            spec = tuple(spec[0])
        out = Layout.from_device_mesh(self._mesh)
        if len(spec) > 0 and isinstance(spec[0], Placement):
            out.set_placements(spec)
            return out
        out._set_alias_map(spec)
        return out

    def _set_alias_map(self, alias_map) -> None:
        names = self._mesh.mesh_dim_names
        used = set()
        dim_axes = []
        for ele in alias_map:
            items = ele if isinstance(ele, (tuple, list)) else (ele,)
            axes = []
            for it in items:
                if it == "None":
                    continue
                if it not in names:
                    raise ValueError(f"The axis {it} is not found in {names}")
                if it in used:
                    raise ValueError(f"The axis {it} has been set more than one in {names}")
                used.add(it)
                axes.append(names.index(it))
            dim_axes.append(tuple(axes))
        self._dim_axes = tuple(dim_axes)
        self._pending_placements = None
        self._compact = None

    # ------------------------------------------------- placement <-> map ---
    def set_placements(self, placements: Sequence[Placement]) -> None:
        placements = tuple(placements)
        # one placement per mesh dim; as in the reference a shorter list leaves the remaining mesh dims
        # replicated and surplus ``Replicate()`` entries are ignored
        nd = self._mesh.ndim
        if len(placements) < nd:
            placements = placements + (Replicate(),) * (nd - len(placements))
        elif len(placements) > nd:
            if any(not isinstance(p, Replicate) for p in placements[nd:]):
                raise ValueError(f"need {nd} placements (one per mesh dim), got {len(placements)}")
            placements = placements[:nd]
        for p in placements:
            if not isinstance(p, Placement):
                raise TypeError(f"expected a Placement, got {p!r}")
        self._pending_placements = placements
        self._partial = [p.reduce_op if isinstance(p, Partial) else None for p in placements]
        self._dim_axes = None
        self._compact = None

    def placement_to_tensor_map(self, ndim: int):
        """Resolve placements against a tensor of ``ndim`` dims; returns ``tensor_map``."""
        if self._pending_placements is None:
            if self._dim_axes is None:
                raise ValueError("layout has neither placements nor a tensor map")
            if len(self._dim_axes) != ndim:
                raise ValueError(f"layout describes {len(self._dim_axes)} dims, tensor has {ndim}")
            return self.tensor_map
        axes: List[List[int]] = [[] for _ in range(ndim)]
        for mi, p in enumerate(self._pending_placements):
            if isinstance(p, Shard):
                d = p.dim + ndim if p.dim < 0 else p.dim
                if not 0 <= d < ndim:
                    raise ValueError(f"Shard(dim={p.dim}) out of range for a {ndim}-D tensor")
                axes[d].append(mi)
        self._dim_axes = tuple(tuple(a) for a in axes)
        self._pending_placements = None
        self._compact = None
        return self.tensor_map

    def tensor_map_to_placement(self) -> Tuple[Placement, ...]:
        return self.placements

    def set_tensor_map(self, tensor_map) -> None:
        nd = self._mesh.ndim
        dim_axes = []
        for m in tensor_map:
            ms = m if isinstance(m, (tuple, list)) else (m,)
            dim_axes.append(tuple(nd - 1 - a for a in ms if a != -1))
        self._dim_axes = tuple(dim_axes)
        self._pending_placements = None
        self._compact = None

    def set_alias_tensor_map(self, alias_map) -> None:
        self._set_alias_map(alias_map)

    def update_compact_str(self) -> None:
        self._compact = None

    # ------------------------------------------------------- properties ---
    @property
    def mesh(self) -> DeviceMesh:
        return self._mesh

    @property
    def mesh_shape(self) -> Tuple[int, ...]:
        return self._mesh.mesh_shape

    @property
    def alias_name(self) -> Tuple[str, ...]:
        return self._mesh.mesh_dim_names

    @property
    def rank_list(self) -> Tuple[int, ...]:
        return self._mesh.rank_list

    @property
    def dim_axes(self) -> DimAxes:
        """Per tensor dim: mesh-dim indices sharding it, outer split first."""
        if self._dim_axes is None:
            raise ValueError("layout is not bound to a tensor rank yet (call placement_to_tensor_map)")
        return self._dim_axes

    @property
    def ndim(self) -> int:
        return len(self.dim_axes)

    @property
    def tensor_map(self):
        if self._dim_axes is None:
            return None
        nd = self._mesh.ndim
        out = []
        for axes in self._dim_axes:
            if not axes:
                out.append(-1)
            elif len(axes) == 1:
                out.append(nd - 1 - axes[0])
            else:
                out.append(tuple(nd - 1 - a for a in axes))
        return tuple(out)

    @property
    def alias_tensor_map(self):
        if self._dim_axes is None:
            return None
        names = self._mesh.mesh_dim_names
        out = []
        for axes in self._dim_axes:
            if not axes:
                out.append("None")
            elif len(axes) == 1:
                out.append(names[axes[0]])
            else:
                out.append(tuple(names[a] for a in axes))
        return tuple(out)

    @property
    def placements(self) -> Optional[Tuple[Placement, ...]]:
        if self._pending_placements is not None:
            return self._pending_placements
        if self._dim_axes is None:
            return None
        res: List[Placement] = [Replicate()] * self._mesh.ndim
        for d, axes in enumerate(self._dim_axes):
            for a in axes:
                res[a] = Shard(d)
        for a, op in enumerate(self._partial):
            if op is not None:
                res[a] = Partial(op)
        return tuple(res)

    @property
    def partial(self) -> List[Optional[str]]:
        return self._partial

    @property
    def sharded_axes(self) -> set:
        return {a for axes in self.dim_axes for a in axes}

    # ---------------------------------------------------------- partial ---
    def _axis_index(self, axis: Union[int, str]) -> int:
        return self._mesh._dim_index(axis)

    def set_partial_by_dev_axis(self, axis: Union[int, str], op: Optional[str]) -> None:
        if op is not None and op not in _PARTIAL_OPS:
            raise ValueError(f"partial op must be one of {_PARTIAL_OPS}, got {op!r}")
        a = self._axis_index(axis)
        if op is not None and self._dim_axes is not None and a in self.sharded_axes:
            raise ValueError(f"mesh axis {self.alias_name[a]!r} shards a tensor dim and cannot also be partial")
        self._partial[a] = op
        self._compact = None

    def get_partial_by_dev_id(self, axis) -> Optional[str]:
        return self._partial[self._axis_index(axis)]

    def reset_partial(self) -> None:
        self._partial = [None] * self._mesh.ndim
        if self._pending_placements is not None:
            self._pending_placements = tuple(Replicate() if isinstance(p, Partial) else p
                                             for p in self._pending_placements)
        self._compact = None

    def is_partial(self) -> bool:
        return any(p is not None for p in self._partial)

    # ------------------------------------------------------------ shapes ---
    def shard_factor(self, dim: int) -> int:
        f = 1
        for a in self.dim_axes[dim]:
            f *= self._mesh.mesh_shape[a]
        return f

    def get_global_shape(self, local_shape: Sequence[int]) -> Tuple[int, ...]:
        if self._dim_axes is None:
            self.placement_to_tensor_map(len(local_shape))
        if len(local_shape) != len(self._dim_axes):
            raise ValueError(f"layout describes {len(self._dim_axes)} dims, shape {tuple(local_shape)} has {len(local_shape)}")
        return tuple(int(n) * self.shard_factor(d) for d, n in enumerate(local_shape))

    def get_local_shape(self, global_shape: Sequence[int]) -> Tuple[int, ...]:
        if self._dim_axes is None:
            self.placement_to_tensor_map(len(global_shape))
        out = []
        for d, n in enumerate(global_shape):
            f = self.shard_factor(d)
            if int(n) % f:
                raise ValueError(f"dim {d} of size {n} is not divisible by {f} (even sharding only)")
            out.append(int(n) // f)
        return tuple(out)

    def repeat_num(self) -> int:
        """Number of ranks of the mesh holding identical data (devices / devices used for sharding)."""
        used = 1
        for a in self.sharded_axes:
            used *= self._mesh.mesh_shape[a]
        return self._mesh.size() // used

    # helper names of the reference's Layout (core/layout.py:447-468, 483-495, 550-580 there)
    def is_dev_axis_apply_shard(self, axis: str) -> bool:
        """Whether the named mesh axis shards some tensor dim."""
        a = self._axis_index(axis)
        return any(a in axes for axes in (self.dim_axes or ()))

    def get_dev_axis_apply_shard_axis(self, axis: str) -> Optional[int]:
        """The tensor dim that the named mesh axis shards, or ``None``."""
        a = self._axis_index(axis)
        for d, axes in enumerate(self.dim_axes or ()):
            if a in axes:
                return d
        return None

    def get_devices_for_axis(self, axis, rank: int):
        """Ranks that differ from ``rank`` only along the named mesh axis."""
        return self._mesh.get_devices_for_axis(axis, rank)

    def to_string(self) -> str:
        """A multi-line dump: mesh shape, axis names, rank list, Partial status and tensor map."""
        tm = "Not configured" if self._dim_axes is None else str(tuple(self.alias_tensor_map))
        return "\n".join((f"Mesh shape: {tuple(self.mesh_shape)}", f"Alias Names: {tuple(self.alias_name)}",
                          f"Rank List: {list(self.rank_list)}", f"Partial: {list(self.partial)}", f"Tensor Map: {tm}"))

    def get_comm_group_by_axis(self, axis):
        return self._mesh.get_group(self._axis_index(axis))

    def slice_area(self, global_shape, rank: Optional[int] = None) -> List[Tuple[int, int]]:
        rank = self._mesh.rank if rank is None else rank
        inner = self.rank_list.index(rank)
        return _infer_slice_area_by_rank(self.mesh_shape, self.tensor_map, inner, global_shape)

    # ---------------------------------------------------------- identity ---
    @property
    def compact_str(self) -> str:
        if self._compact is None:
            self._compact = f"{self._mesh.to_hash()}|{self.tensor_map}|{self._partial}"
        return self._compact

    def to_dict(self) -> dict:
        if self._dim_axes is None:
            raise ValueError("The tensor_map of layout is None")
        return {"mesh_shape": self.mesh_shape, "tensor_map": self.tensor_map,
                "interleaved_parallel": "interleaved_parallel" in self.alias_name,
                "alias_name": self.alias_name, "rank_list": self.rank_list}

    def __eq__(self, other):
        if not isinstance(other, Layout):
            return NotImplemented
        return (self._mesh == other._mesh and self._dim_axes == other._dim_axes
                and self._partial == other._partial
                and (self._dim_axes is not None or self._pending_placements == other._pending_placements))

    def __hash__(self):
        return hash((self._mesh.to_hash(), self._dim_axes, tuple(self._partial)))

    def __repr__(self):
        return (f"Layout(mesh_shape={self.mesh_shape}, alias_name={self.alias_name}, "
                f"tensor_map={self.tensor_map}, partial={self._partial}, rank_list={list(self.rank_list)})")
