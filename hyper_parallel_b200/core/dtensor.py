"""``DTensor``: a ``torch.Tensor`` subclass that pairs a local shard with a layout.

Semantics follow hyper_parallel/core/dtensor.py:85-486 and
hyper_parallel/platform/torch/dtensor.py:21-232 of the reference:

* the subclass instance aliases the storage of the local shard, autograd runs on
  the **local** tensor, and ``grad / requires_grad / is_leaf / backward`` forward to it;
* ``.shape`` / ``.size()`` / ``.numel()`` are **global**, ``.local_shape`` /
  ``.to_local()`` are local;
* every ``torch`` function called on a DTensor is routed to the distributed-op
  dispatcher, which infers the output layout from the input layouts.

``DTensor.from_local(local, mesh, placements)`` and the README spelling
``DTensor.from_local(local, layout)`` are both accepted.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence, Tuple

import torch

from .device_mesh import DeviceMesh
from .layout import Layout, _get_slice_tensor_by_layout
from .placement_types import Placement, Replicate

_LAYOUT_CACHE: Dict[tuple, Layout] = {}
_DISPATCH_ENABLED = True


def _dispatch_enabled() -> bool:
    return _DISPATCH_ENABLED


class SkipDTensorDispatch:
    """Context manager: inside it torch functions see DTensors as their local tensors.

    Used around ``optimizer.step()`` so that optimizers update the local shards directly.
    """

    def __enter__(self):
        global _DISPATCH_ENABLED
        self._prev = _DISPATCH_ENABLED
        _DISPATCH_ENABLED = False
        return self

    def __exit__(self, *exc):
        global _DISPATCH_ENABLED
        _DISPATCH_ENABLED = self._prev
        return False


def _build_layout(device_mesh: DeviceMesh, placements: Sequence[Placement], ndim: int) -> Layout:
    key = (device_mesh.to_hash(), tuple(placements), ndim)
    lay = _LAYOUT_CACHE.get(key)
    if lay is None:
        given = tuple(placements) or (Replicate(),) * device_mesh.ndim      # none given: replicated everywhere
        lay = Layout.from_device_mesh(device_mesh)(given)
        lay.placement_to_tensor_map(ndim)
        _LAYOUT_CACHE[key] = lay
    return lay


class DTensor(torch.Tensor):
    """Distributed tensor = local shard + device mesh + placements."""

    _local_tensor: torch.Tensor
    _layout: Layout

    @staticmethod
    def __new__(cls, local_tensor, device_mesh=None, placements=None):
        if isinstance(local_tensor, DTensor):
            src = local_tensor
            t = torch.Tensor._make_subclass(cls, src._local_tensor, src._local_tensor.requires_grad)
            t._local_tensor = src._local_tensor
            t._layout = src._layout
            return t
        if isinstance(device_mesh, Layout):
            layout = device_mesh
            if layout._dim_axes is None:
                layout = layout.copy()
                layout.placement_to_tensor_map(local_tensor.dim())
        else:
            if device_mesh is None:
                raise ValueError("device_mesh is None, must provide a DeviceMesh instance")
            if placements is None:
                raise ValueError("placements is None, must provide placements")
            layout = _build_layout(device_mesh, placements, local_tensor.dim())
        return cls._wrap(local_tensor, layout)

    @classmethod
    def _wrap(cls, local_tensor: torch.Tensor, layout: Layout) -> "DTensor":
        """Fast path used by the dispatcher: ``layout`` is already bound to the tensor rank."""
        t = torch.Tensor._make_subclass(cls, local_tensor, local_tensor.requires_grad)
        t._local_tensor = local_tensor
        t._layout = layout
        return t

    # ------------------------------------------------------------ dispatch --
    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        from .shard._op_dispatch import _OP_DISPATCHER
        return _OP_DISPATCHER.dispatch(func, args, kwargs or {})

    # -------------------------------------------------------- constructors --
    @staticmethod
    def from_local(local_tensor: torch.Tensor, device_mesh, placements=None) -> "DTensor":
        return DTensor(local_tensor, device_mesh, placements)

    def to_local(self) -> torch.Tensor:
        return self._local_tensor

    # ------------------------------------------------------------ metadata --
    @property
    def device_mesh(self) -> DeviceMesh:
        return self._layout.mesh

    @property
    def placements(self) -> Tuple[Placement, ...]:
        return self._layout.placements

    @property
    def layout(self) -> Layout:
        return self.__dict__.get("_layout")

    @property
    def shape(self):
        return torch.Size(self._layout.get_global_shape(self._local_tensor.shape))

    def size(self, dim: Optional[int] = None):
        s = self.shape
        return s if dim is None else s[dim]

    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    @property
    def local_shape(self):
        return self._local_tensor.shape

    @property
    def ndim(self) -> int:
        return self._local_tensor.dim()

    def dim(self) -> int:
        return self._local_tensor.dim()

    @property
    def device(self):
        return self._local_tensor.device

    @property
    def dtype(self):
        return self._local_tensor.dtype

    def data_ptr(self) -> int:
        return self._local_tensor.data_ptr()

    def element_size(self) -> int:
        return self._local_tensor.element_size()

    def is_contiguous(self, *a, **k) -> bool:
        return self._local_tensor.is_contiguous(*a, **k)

    # ------------------------------------------------------------- autograd --
    @property
    def grad(self):
        return self._local_tensor.grad

    @grad.setter
    def grad(self, value):
        if isinstance(value, DTensor):
            value = value._local_tensor
        self._local_tensor.grad = value

    def grad_zero_(self):
        """Zero the local gradient in place (reference platform/torch/dtensor.py:108-111)."""
        if self._local_tensor.grad is not None:
            g = self._local_tensor.grad
            (g._local_tensor if isinstance(g, DTensor) else g).zero_()
        return self

    @property
    def requires_grad(self) -> bool:
        return self._local_tensor.requires_grad

    @requires_grad.setter
    def requires_grad(self, value: bool):
        self.requires_grad_(value)

    def requires_grad_(self, requires_grad: bool = True):
        self._local_tensor.requires_grad_(requires_grad)
        with torch._C.DisableTorchFunctionSubclass():
            if torch.Tensor.is_leaf.__get__(self):
                torch.Tensor.requires_grad_(self, requires_grad)
        return self

    @property
    def grad_fn(self):
        return self._local_tensor.grad_fn

    @property
    def is_leaf(self) -> bool:
        return self._local_tensor.is_leaf

    @property
    def retains_grad(self) -> bool:
        return self._local_tensor.retains_grad

    def retain_grad(self):
        self._local_tensor.retain_grad()

    def backward(self, gradient=None, retain_graph=None, create_graph=False, inputs=None):
        if isinstance(gradient, DTensor):
            gradient = gradient._local_tensor
        self._local_tensor.backward(gradient, retain_graph, create_graph, inputs=inputs)

    def register_hook(self, hook):
        return self._local_tensor.register_hook(hook)

    def detach(self):
        return DTensor._wrap(self._local_tensor.detach(), self._layout)

    def detach_(self):
        self._local_tensor.detach_()
        return self

    @property
    def data(self):
        return DTensor._wrap(self._local_tensor.data, self._layout)

    @data.setter
    def data(self, value):
        if isinstance(value, DTensor):
            value = value._local_tensor
        self._rebind(value.detach().requires_grad_(self._local_tensor.requires_grad))

    # --------------------------------------------------------- conversions --
    def to(self, *args, **kwargs):
        return DTensor._wrap(self._local_tensor.to(*args, **kwargs), self._layout)

    def type(self, dtype=None, non_blocking=False):
        if dtype is None:
            return self._local_tensor.type()
        return DTensor._wrap(self._local_tensor.to(dtype=dtype, non_blocking=non_blocking), self._layout)

    def cpu(self):
        return DTensor._wrap(self._local_tensor.cpu(), self._layout)

    def cuda(self, *a, **k):
        return DTensor._wrap(self._local_tensor.cuda(*a, **k), self._layout)

    def item(self):
        return self._local_tensor.item()

    def tolist(self):
        return self._local_tensor.tolist()

    def numpy(self):
        return self._local_tensor.detach().cpu().numpy()

    # ------------------------------------------------- in-place data rebind --
    def _rebind(self, new_local: torch.Tensor) -> None:
        """Point this DTensor at a new local tensor (used when a leaf parameter is re-initialised)."""
        with torch.no_grad(), torch._C.DisableTorchFunctionSubclass():
            torch.Tensor.set_(self, new_local.detach())
        self._local_tensor = new_local

    def _inplace(self, fn_name, *args, **kwargs):
        args = tuple(a._local_tensor if isinstance(a, DTensor) else a for a in args)
        lt = self._local_tensor
        if lt.requires_grad and lt.is_leaf and torch.is_grad_enabled():
            with torch.no_grad():
                getattr(lt, fn_name)(*args, **kwargs)
        else:
            getattr(lt, fn_name)(*args, **kwargs)
        return self

    def zero_(self):
        return self._inplace("zero_")

    def fill_(self, value):
        return self._inplace("fill_", value)

    def copy_(self, src, non_blocking: bool = False):
        return self._inplace("copy_", src, non_blocking=non_blocking)

    # ------------------------------------------------------ redistribution --
    def redistribute(self, device_mesh, placements=None) -> "DTensor":
        """Return this tensor re-laid-out as ``placements`` on ``device_mesh`` (or as a ``Layout``)."""
        from .tensor_redistribution import _tensor_redistribution
        if isinstance(device_mesh, Layout):
            dst = device_mesh
            if dst._dim_axes is None:
                dst = dst.copy()
                dst.placement_to_tensor_map(self._local_tensor.dim())
        else:
            dst = _build_layout(device_mesh, placements, self._local_tensor.dim())
        return _tensor_redistribution.redistribution(self, dst)

    def reduce_partial(self) -> "DTensor":
        """Resolve every pending reduction (all-reduce over the partial mesh axes)."""
        if not self._layout.is_partial():
            return self
        from .tensor_redistribution import _tensor_redistribution
        dst = self._layout.copy()
        dst.reset_partial()
        return _tensor_redistribution.redistribution(self, dst)

    def full_tensor(self) -> torch.Tensor:
        """Gather the complete (global) tensor on every rank of the mesh."""
        mesh = self._layout.mesh
        dst = _build_layout(mesh, (Replicate(),) * mesh.ndim, self._local_tensor.dim())
        from .tensor_redistribution import _tensor_redistribution
        return _tensor_redistribution.redistribution(self, dst)._local_tensor

    def __repr__(self):
        return (f"DTensor(local_tensor={self._local_tensor}, device_mesh={self._layout.mesh}, "
                f"placements={self._layout.placements})")

    def __format__(self, spec):
        return self._local_tensor.__format__(spec)

    def __reduce_ex__(self, proto):
        return (_rebuild_dtensor, (self._local_tensor, self._layout.mesh.mesh_shape,
                                   self._layout.mesh.mesh_dim_names, self._layout.mesh.rank_list,
                                   self._layout.placements))

    def __deepcopy__(self, memo):
        new_local = self._local_tensor.detach().clone().requires_grad_(self._local_tensor.requires_grad)
        out = DTensor._wrap(new_local, self._layout)
        memo[id(self)] = out
        return out


def _rebuild_dtensor(local, mesh_shape, names, rank_list, placements):
    from .device_mesh import _create_device_mesh
    mesh = _create_device_mesh("cuda", mesh_shape, mesh_dim_names=names, rank_list=rank_list,
                               init_backend=False)
    return DTensor(local, mesh, placements)


# ------------------------------------------------------------------ factories --
def distribute_tensor(tensor: torch.Tensor, device_mesh, placements=None) -> DTensor:
    """Slice a replicated global ``tensor`` into this rank's shard (no communication)."""
    if isinstance(device_mesh, Layout):
        layout = device_mesh.copy()
        layout.placement_to_tensor_map(tensor.dim())
    else:
        layout = _build_layout(device_mesh, placements, tensor.dim())
    if layout.is_partial():
        raise ValueError("distribute_tensor cannot create a Partial tensor")
    local = _get_slice_tensor_by_layout(tensor.detach(), layout).requires_grad_(tensor.requires_grad)
    return DTensor._wrap(local, layout)


def _factory(fn, size, device_mesh, placements, **kwargs) -> DTensor:
    if isinstance(size, int):
        size = (size,)
    size = tuple(size)
    layout = _build_layout(device_mesh, placements, len(size))
    return DTensor._wrap(fn(compute_local_shape(size, layout), **kwargs), layout)


def compute_local_shape_and_offset(global_shape, layout: Layout) -> Tuple[Tuple[int, ...], Tuple[int, ...]]:
    """This rank's shard shape of a tensor of ``global_shape`` under ``layout`` and where the shard
    starts in the global tensor, with ``torch.chunk`` semantics where a dimension does not divide
    evenly: chunks of ``ceil(n / parts)``, a shorter last one, empty ones after it (their start is the
    end of the data).  The factory functions use it (reference dtensor.py:334-369,
    ``compute_local_shape_and_global_offset``); the layout algebra itself (``shape``,
    redistribution) assumes even shards, as the reference's does."""
    from .random import local_shard_size_and_offset
    mesh = layout.mesh
    coord = mesh.get_coordinate()
    shape, offset = [], []
    for d, n in enumerate(global_shape):
        n, start = int(n), 0
        for a in layout.dim_axes[d]:
            n, off = local_shard_size_and_offset(n, mesh.mesh_shape[a], coord[a])
            start += off
        shape.append(n)
        offset.append(start)
    return tuple(shape), tuple(offset)


def compute_local_shape(global_shape, layout: Layout) -> Tuple[int, ...]:
    return compute_local_shape_and_offset(global_shape, layout)[0]


def ones(size, device_mesh=None, placements=None, **kwargs) -> DTensor:
    return _factory(torch.ones, size, device_mesh, placements, **kwargs)


def zeros(size, device_mesh=None, placements=None, **kwargs) -> DTensor:
    return _factory(torch.zeros, size, device_mesh, placements, **kwargs)


def empty(size, device_mesh=None, placements=None, **kwargs) -> DTensor:
    return _factory(torch.empty, size, device_mesh, placements, **kwargs)


def full(size, fill_value, *, device_mesh=None, placements=None, **kwargs) -> DTensor:
    return _factory(lambda s, **kw: torch.full(s, fill_value, **kw), size, device_mesh, placements, **kwargs)
