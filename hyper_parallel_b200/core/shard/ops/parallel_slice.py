"""Slicing: ``x[...]`` (basic indexing), ``narrow``, ``select``.  A dim that is only partly kept
must be unsharded; fully kept dims keep their sharding
(hyper_parallel/core/shard/ops/parallel_slice.py:22-76, parallel_slice_ext.py:22-46)."""
from __future__ import annotations

import torch

from ._common import make, norm_dim, split_shapes
from .parallel_ops import DistributedOp


class SliceDistributedOp(DistributedOp):
    _with_shape_convention = True     # called in the "WithShape" form although registered as "Slice"

    _allow_partial_inputs = True

    def infer_layout(self, layouts, extra_args):
        x = layouts[0]
        extra, shapes = split_shapes(extra_args)
        shape = shapes[0]
        nd = len(shape)
        if self.op_name == "narrow":
            dim, start, length = norm_dim(extra[0], nd), extra[1], extra[2]
            if x.dim_axes[dim] and not (start == 0 and length == shape[dim]):
                raise ValueError(f"For narrow, partially sliced dim {dim} must not be sharded")
            return make(x, x.dim_axes, x.partial)
        if self.op_name == "select":
            dim = norm_dim(extra[0], nd)
            if x.dim_axes[dim]:
                raise ValueError(f"For select, dim {dim} must not be sharded")
            return make(x, [a for d, a in enumerate(x.dim_axes) if d != dim], x.partial)
        # __getitem__
        index = extra[0] if extra else ()
        if not isinstance(index, tuple):
            index = (index,)
        n_specified = sum(1 for i in index if i is not None and i is not Ellipsis)
        out = []
        d = 0
        for it in index:
            if it is None:
                out.append(())
            elif it is Ellipsis:
                for _ in range(nd - n_specified):
                    out.append(x.dim_axes[d]); d += 1
            elif isinstance(it, slice):
                full = it == slice(None) or (it.start in (None, 0) and it.stop in (None, shape[d])
                                             and it.step in (None, 1))
                if not full and x.dim_axes[d]:
                    raise ValueError(f"For indexing, partially sliced dim {d} must not be sharded")
                out.append(x.dim_axes[d] if full else ()); d += 1
            elif isinstance(it, int):
                if x.dim_axes[d]:
                    raise ValueError(f"For indexing, dim {d} selected by an int must not be sharded")
                d += 1
            elif isinstance(it, torch.Tensor):
                raise ValueError("advanced (tensor) indexing of a DTensor is not supported; "
                                 "use index_select / gather")
            else:
                raise ValueError(f"unsupported index element {it!r}")
        while d < nd:
            out.append(x.dim_axes[d]); d += 1
        return make(x, out, x.partial)


SliceExtDistributedOp = SliceDistributedOp
