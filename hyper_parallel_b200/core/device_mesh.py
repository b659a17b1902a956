"""n-dimensional grid of ranks with one process group per mesh dimension.

Capabilities follow hyper_parallel/core/device_mesh.py:68-1079 of the reference:
row-major rank order (last mesh dim varies fastest), named dims, sub-mesh slicing
(``mesh["tp"]``, ``mesh["dp", "tp"]``), ``flatten``, ``from_group``, per-dim groups,
local ranks / coordinates, and ``init_device_mesh`` whose default rank list is the
aligned block of ranks that contains the caller (so that each pipeline stage can
build its own mesh).  Rank lists per dimension are computed with array slicing
rather than by enumerating every rank's sub-list.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from ..collectives import cc

_DEVICE_MESH_CACHE: Dict[tuple, "DeviceMesh"] = {}


def _as_array(mesh) -> np.ndarray:
    if isinstance(mesh, torch.Tensor):
        arr = mesh.detach().cpu().numpy()
    else:
        arr = np.asarray(mesh)
    if arr.ndim == 0:
        arr = arr.reshape(1)
    return arr.astype(np.int64)


class DeviceMesh:
    """A named n-D arrangement of global ranks.

    Args:
        device_type: ``"cuda"``, ``"cpu"`` (``"npu"`` is accepted and ignored so that
            scripts written for the reference run unchanged).
        mesh: nested list / array / tensor of global ranks, **or** a mesh shape tuple
            together with ``rank_list``.
        mesh_dim_names: one name per mesh dimension.
        rank_list: flat list of ranks when ``mesh`` is a shape.
        _init_backend: create the per-dimension process groups now.
        _rank: pretend to be this rank (layout arithmetic without a process group).
    """

    def __init__(self, device_type: str, mesh, *, mesh_dim_names: Optional[Sequence[str]] = None,
                 rank_list: Optional[Sequence[int]] = None, _init_backend: bool = True,
                 _rank: Optional[int] = None, _root: Optional["DeviceMesh"] = None):
        self.device_type = device_type
        if rank_list is not None:
            shape = tuple(int(s) for s in mesh)
            arr = np.asarray(list(rank_list), dtype=np.int64).reshape(shape)
        else:
            arr = _as_array(mesh)
        self._mesh = arr
        self._shape: Tuple[int, ...] = tuple(int(s) for s in arr.shape)
        if mesh_dim_names is None:
            mesh_dim_names = tuple(f"dim{i}" for i in range(arr.ndim))
        mesh_dim_names = tuple(mesh_dim_names)
        if len(mesh_dim_names) != arr.ndim:
            raise ValueError(f"mesh_dim_names {mesh_dim_names} does not match mesh of {arr.ndim} dims")
        if len(set(mesh_dim_names)) != len(mesh_dim_names):
            raise ValueError(f"mesh_dim_names must be unique, got {mesh_dim_names}")
        if "interleaved_parallel" in mesh_dim_names[:-1]:
            raise ValueError('"interleaved_parallel" is reserved for the last mesh dimension')
        self._dim_names = mesh_dim_names
        flat = arr.reshape(-1)
        if len(set(flat.tolist())) != flat.size:
            raise ValueError("mesh contains duplicate ranks")
        self._rank_list: Tuple[int, ...] = tuple(int(r) for r in flat)
        self._rank = cc.get_rank() if _rank is None else int(_rank)
        self._root = _root
        self._sub_cache: Dict[tuple, "DeviceMesh"] = {}
        self._flatten_cache: Dict[str, "DeviceMesh"] = {}
        self._groups: List[Optional[object]] = [None] * arr.ndim
        self._groups_ready = False
        pos = np.argwhere(arr == self._rank)
        self._coord: Optional[Tuple[int, ...]] = tuple(int(c) for c in pos[0]) if len(pos) else None
        self._hash = hash((self._shape, self._rank_list, self._dim_names))
        if _init_backend:
            self._init_groups()

    # ------------------------------------------------------------ groups --
    def _init_groups(self) -> None:
        if self._groups_ready or not cc.is_initialized() or self._coord is None:
            self._groups_ready = self._groups_ready or not cc.is_initialized()
            return
        for d in range(self.ndim):
            ranks = self.get_rank_list_along_axis(d)
            # an axis of size one gets a real one-member group: ``None`` would mean the world
            self._groups[d] = cc.group_for_ranks(ranks) if len(ranks) > 1 else cc.self_group()
        self._groups_ready = True

    def get_rank_list_along_axis(self, dim: Union[int, str]) -> List[int]:
        """Ranks that differ from this rank only in mesh dimension ``dim`` (in mesh order)."""
        d = self._dim_index(dim)
        if self._coord is None:
            raise RuntimeError(f"rank {self._rank} is not part of mesh {self._rank_list}")
        idx = list(self._coord)
        idx[d] = slice(None)
        return [int(r) for r in self._mesh[tuple(idx)]]

    def get_group(self, dim: Union[int, str, None] = None):
        """Process group of mesh dimension ``dim`` (the only dimension of a 1-D mesh by default)."""
        if dim is None:
            if self.ndim != 1:
                raise RuntimeError("get_group() without a dim needs a 1-D mesh")
            dim = 0
        d = self._dim_index(dim)
        if not self._groups_ready:
            self._init_groups()
        return self._groups[d]

    def get_comm_group_by_axis(self, dim):
        return self.get_group(dim)

    # names of the reference's helpers (core/device_mesh.py:320-327, 751-769, 905-969 there)
    def axis_index(self, axis: str) -> int:
        """Position of the named dim in ``mesh_shape``."""
        if axis not in self._dim_names:
            raise ValueError(f"The axis name must be one of mesh dim names {self._dim_names}, but got {axis}")
        return self._dim_names.index(axis)

    def axis_id(self, axis: str) -> int:
        """The number a ``tensor_map`` uses for the named dim (dims count from the last one; "None" is -1)."""
        if axis == "None":
            return -1
        return self.ndim - 1 - self.axis_index(axis)

    def get_devices_for_axis(self, mesh_dim: Union[str, int], rank: int) -> List[int]:
        """Ranks that differ from ``rank`` only in mesh dimension ``mesh_dim`` (any member rank)."""
        if isinstance(mesh_dim, str) and mesh_dim not in self._dim_names:
            raise ValueError(f"mesh_dim '{mesh_dim}' not found in mesh_dim_names {self._dim_names}")
        if not isinstance(mesh_dim, str) and not 0 <= int(mesh_dim) < self.ndim:
            raise ValueError(f"mesh_dim {mesh_dim} can not out of range [0, {self.ndim})")
        d = self._dim_index(mesh_dim)
        idx = list(self.coordinate_of(int(rank)))
        idx[d] = slice(None)
        return [int(r) for r in self._mesh[tuple(idx)]]

    def get_flatten_mapping(self) -> Dict[str, "DeviceMesh"]:
        """``{name: 1-D mesh}`` of the ``flatten()`` calls registered on this (root) mesh."""
        return self.root_mesh._flatten_cache

    def add_flatten_mapping(self, name: str, mesh: "DeviceMesh") -> None:
        self.root_mesh._flatten_cache[name] = mesh

    # ----------------------------------------------------------- queries --
    def _dim_index(self, dim: Union[int, str]) -> int:
        if isinstance(dim, str):
            if dim not in self._dim_names:
                raise KeyError(f"mesh dim {dim!r} not in {self._dim_names}")
            return self._dim_names.index(dim)
        d = int(dim)
        if d < 0:
            d += self.ndim
        if not 0 <= d < self.ndim:
            raise IndexError(f"mesh dim {dim} out of range for {self.ndim}-D mesh")
        return d

    @property
    def mesh(self) -> torch.Tensor:
        return torch.from_numpy(self._mesh.copy()).to(torch.int32)

    @property
    def mesh_shape(self) -> Tuple[int, ...]:
        return self._shape

    @property
    def mesh_dim_names(self) -> Tuple[str, ...]:
        return self._dim_names

    @property
    def rank_list(self) -> Tuple[int, ...]:
        return self._rank_list

    @property
    def rank(self) -> int:
        return self._rank

    @property
    def ndim(self) -> int:
        return len(self._shape)

    @property
    def root_mesh(self) -> "DeviceMesh":
        return self._root if self._root is not None else self

    @property
    def sub_mesh(self) -> Dict[tuple, "DeviceMesh"]:
        return self._sub_cache

    def size(self, dim: Union[int, str, None] = None) -> int:
        if dim is None:
            return int(np.prod(self._shape))
        return self._shape[self._dim_index(dim)]

    def get_device_num_along_axis(self, dim) -> int:
        return self.size(dim)

    def get_local_rank(self, dim: Union[int, str, None] = None) -> int:
        """Index of this rank along mesh dimension ``dim``."""
        if dim is None:
            if self.ndim != 1:
                raise RuntimeError("get_local_rank() without a dim needs a 1-D mesh")
            dim = 0
        if self._coord is None:
            raise RuntimeError(f"rank {self._rank} is not part of this mesh")
        return self._coord[self._dim_index(dim)]

    def get_coordinate(self) -> Optional[Tuple[int, ...]]:
        return self._coord

    def coordinate_of(self, rank: int) -> Tuple[int, ...]:
        """Mesh coordinate of any member rank."""
        pos = np.argwhere(self._mesh == rank)
        if not len(pos):
            raise ValueError(f"rank {rank} is not part of mesh {self._rank_list}")
        return tuple(int(c) for c in pos[0])

    def get_global_shape(self, slice_shape: Sequence[int], tensor_map: Sequence) -> Tuple[int, ...]:
        """Global shape from a local shape and a reference-style ``tensor_map``
        (``-1`` or reversed mesh-dim index, or tuples of them)."""
        out = []
        for n, m in zip(slice_shape, tensor_map):
            ms = m if isinstance(m, (tuple, list)) else (m,)
            f = 1
            for a in ms:
                if a != -1:
                    f *= self._shape[self.ndim - 1 - a]
            out.append(int(n) * f)
        return tuple(out)

    def to_hash(self) -> int:
        return self._hash

    def __hash__(self):
        return self._hash

    def __eq__(self, other):
        return (isinstance(other, DeviceMesh) and self._shape == other._shape
                and self._rank_list == other._rank_list and self._dim_names == other._dim_names)

    def __repr__(self):
        return (f"DeviceMesh({self.device_type!r}, shape={self._shape}, names={self._dim_names}, "
                f"ranks={list(self._rank_list)})")

    # ---------------------------------------------------------- sub-mesh --
    def __getitem__(self, names: Union[str, Sequence[str]]) -> "DeviceMesh":
        """Sub-mesh over the named dims that contains this rank (other dims fixed at its coordinate)."""
        if isinstance(names, str):
            names = (names,)
        names = tuple(names)
        if names in self._sub_cache:
            return self._sub_cache[names]
        if len(names) == 1 and names[0] not in self._dim_names and names[0] in self.root_mesh._flatten_cache:
            return self.root_mesh._flatten_cache[names[0]]        # the name of an earlier ``flatten()``
        dims = [self._dim_index(n) for n in names]
        if len(set(dims)) != len(dims):
            raise KeyError(f"duplicate mesh dims in {names}")
        if dims != sorted(dims):
            raise KeyError(f"sub-mesh dims must keep mesh order, got {names} of {self._dim_names}")
        if self._coord is None:
            raise RuntimeError(f"rank {self._rank} is not part of this mesh")
        idx = [self._coord[d] if d not in dims else slice(None) for d in range(self.ndim)]
        sub = DeviceMesh(self.device_type, self._mesh[tuple(idx)], mesh_dim_names=names,
                         _init_backend=False, _rank=self._rank, _root=self.root_mesh)
        # share the parent's communicators instead of creating new ones
        if self._groups_ready or cc.is_initialized():
            self._init_groups()
            sub._groups = [self._groups[d] for d in dims]
            sub._groups_ready = True
        self._sub_cache[names] = sub
        return sub

    def flatten(self, mesh_dim_name: Optional[str] = None) -> "DeviceMesh":
        """Collapse this (sub-)mesh into a 1-D mesh with its own group, registered on the root."""
        name = mesh_dim_name or "_".join(self._dim_names)
        root = self.root_mesh
        if name in root._flatten_cache:
            return root._flatten_cache[name]
        flat = DeviceMesh(self.device_type, self._mesh.reshape(-1), mesh_dim_names=(name,),
                          _init_backend=True, _rank=self._rank, _root=root)
        root._flatten_cache[name] = flat
        return flat

    @staticmethod
    def from_group(group, device_type: str, mesh=None, *, mesh_dim_names=None) -> "DeviceMesh":
        """Build a mesh around existing process group(s)."""
        groups = list(group) if isinstance(group, (list, tuple)) else [group]
        if len(groups) == 1 and mesh is None:
            ranks = cc.get_process_group_ranks(groups[0])
            dm = DeviceMesh(device_type, ranks, mesh_dim_names=mesh_dim_names, _init_backend=False)
            dm._groups = [groups[0]]
            dm._groups_ready = True
            for r in [tuple(ranks)]:
                cc._GROUP_CACHE.setdefault(r, groups[0])
            return dm
        if mesh is None:
            raise ValueError("an n-D mesh must be given together with several groups")
        dm = DeviceMesh(device_type, mesh, mesh_dim_names=mesh_dim_names, _init_backend=False)
        if len(groups) != dm.ndim:
            raise ValueError(f"expected {dm.ndim} groups, got {len(groups)}")
        for d, g in enumerate(groups):
            expect = dm.get_rank_list_along_axis(d)
            got = cc.get_process_group_ranks(g)
            if list(expect) != list(got):
                raise ValueError(f"group for dim {d} has ranks {got}, mesh expects {expect}")
        dm._groups = groups
        dm._groups_ready = True
        return dm


def _create_device_mesh(device_type, mesh_shape, *, mesh_dim_names=None, rank_list=None,
                        init_backend=True, rank=None) -> DeviceMesh:
    mesh_shape = tuple(int(s) for s in mesh_shape)
    n = int(np.prod(mesh_shape))
    if rank_list is None:
        rank_list = tuple(range(n))
    rank_list = tuple(int(r) for r in rank_list)
    if len(rank_list) != n:
        raise ValueError(f"rank_list has {len(rank_list)} entries, mesh_shape {mesh_shape} needs {n}")
    names = tuple(mesh_dim_names) if mesh_dim_names is not None else None
    key = (mesh_shape, names, rank_list, cc.get_rank() if rank is None else rank)
    dm = _DEVICE_MESH_CACHE.get(key)
    if dm is None:
        dm = DeviceMesh(device_type, mesh_shape, mesh_dim_names=names, rank_list=rank_list,
                        _init_backend=init_backend, _rank=rank)
        _DEVICE_MESH_CACHE[key] = dm
    elif init_backend:
        dm._init_groups()
    return dm


def init_device_mesh(device_type: str, mesh_shape: Sequence[int], *,
                     mesh_dim_names: Optional[Sequence[str]] = None,
                     rank_list: Optional[Sequence[int]] = None,
                     init_backend: bool = True) -> DeviceMesh:
    """Create (or fetch from the cache) a mesh of ``mesh_shape``.

    Without ``rank_list`` the mesh covers the aligned block of ``prod(mesh_shape)``
    consecutive ranks that contains the calling rank: with 8 ranks and shape (2, 2),
    ranks 0-3 get the mesh [0..3] and ranks 4-7 get [4..7].
    """
    if init_backend and not cc.is_initialized() and cc.get_world_size() == 1:
        import os
        if "RANK" in os.environ and "WORLD_SIZE" in os.environ:
            cc.init_process_group()
    if rank_list is None:
        n = int(np.prod(tuple(mesh_shape)))
        base = (cc.get_rank() // n) * n
        rank_list = tuple(range(base, base + n))
    return _create_device_mesh(device_type, mesh_shape, mesh_dim_names=mesh_dim_names,
                               rank_list=rank_list, init_backend=init_backend)


def clear_mesh_cache() -> None:
    """Forget every cached mesh (tests use this between cases)."""
    _DEVICE_MESH_CACHE.clear()
