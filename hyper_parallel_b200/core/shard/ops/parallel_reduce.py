"""Layout rules for reductions (``sum mean prod all any max min amax amin argmax argmin``).

As in hyper_parallel/core/shard/ops/parallel_reduce.py:31-311 of the reference: a
reduced dim that is sharded turns into a pending reduction (``Partial``) on its
mesh axes (``sum``, ``avg`` for mean, ``prod``, ``all``, ``max``, ``min``; ``any`` is a ``max`` over
booleans);
``max/min`` with a ``dim`` return ``(values, indices)`` and need that dim unsharded,
as do ``argmax/argmin``.
"""
from __future__ import annotations

from ._common import make, norm_dims, require_unsharded
from .parallel_ops import DistributedOp

_PARTIAL_OF = {"sum": "sum", "mean": "avg", "prod": "prod", "all": "all", "max": "max", "min": "min",
               "amax": "max", "amin": "min", "any": "max", "nansum": "sum"}


def _parse_dim_keepdim(extra_args, ndim):
    dims, keepdim = None, False
    rest = [a for a in extra_args if not isinstance(a, (type(None),)) ]
    for a in rest:
        if isinstance(a, bool):
            keepdim = a
        elif isinstance(a, int):
            if dims is None:
                dims = [a]
        elif isinstance(a, (list, tuple)) and all(isinstance(i, int) for i in a):
            if dims is None:
                dims = list(a)
    return (norm_dims(dims, ndim) if dims is not None and len(dims) > 0 else list(range(ndim))), keepdim, dims is not None


class ReduceExtDistributedOpBase(DistributedOp):
    partial_op = "sum"

    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        x = layouts[0]
        nd = len(x.dim_axes)
        dims, keepdim, _ = _parse_dim_keepdim(extra_args, nd)
        op = _PARTIAL_OF.get(self.op_name, self.partial_op)
        partial = [None] * x.mesh.ndim
        out_axes = []
        for d, axes in enumerate(x.dim_axes):
            if d in dims:
                if axes and op is None:
                    raise ValueError(f"For {self.op_name}, reduced dim {d} must not be sharded")
                for a in axes:
                    partial[a] = op
                if keepdim:
                    out_axes.append(())
            else:
                out_axes.append(axes)
        return make(x, out_axes, partial)


class SumExtDistributedOp(ReduceExtDistributedOpBase):
    partial_op = "sum"


class MeanExtDistributedOp(ReduceExtDistributedOpBase):
    partial_op = "avg"


class ProdExtDistributedOp(ReduceExtDistributedOpBase):
    partial_op = "prod"


class AllExtDistributedOp(ReduceExtDistributedOpBase):
    partial_op = "all"


class ReduceMaxDistributedOp(ReduceExtDistributedOpBase):
    partial_op = "max"


class MaxDistributedOp(DistributedOp):
    """``max/min``: full reduction -> Partial(max/min); with ``dim`` -> (values, indices)."""

    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        x = layouts[0]
        if len(layouts) > 1 and layouts[1] is not None:
            from .parallel_elementwise import ElementWiseDistributedOp
            return ElementWiseDistributedOp.infer_layout(self, layouts, extra_args)
        nd = len(x.dim_axes)
        dims, keepdim, given = _parse_dim_keepdim(extra_args, nd)
        op = "max" if "max" in self.op_name else "min"
        if not given:
            partial = [None] * x.mesh.ndim
            for axes in x.dim_axes:
                for a in axes:
                    partial[a] = op
            return make(x, [], partial)
        require_unsharded(self.op_name, x, dims, "reduced")
        out_axes = [(() if d in dims else axes) for d, axes in enumerate(x.dim_axes) if keepdim or d not in dims]
        lay = make(x, out_axes)
        return (lay, lay)


class ArgMaxWithValueDistributedOp(DistributedOp):
    """``argmax/argmin``: the reduced dim must be unsharded."""

    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        x = layouts[0]
        nd = len(x.dim_axes)
        dims, keepdim, given = _parse_dim_keepdim(extra_args, nd)
        if not given:
            require_unsharded(self.op_name, x, range(nd), "flattened")
            return make(x, [])
        require_unsharded(self.op_name, x, dims, "reduced")
        out_axes = [(() if d in dims else axes) for d, axes in enumerate(x.dim_axes) if keepdim or d not in dims]
        return make(x, out_axes)
