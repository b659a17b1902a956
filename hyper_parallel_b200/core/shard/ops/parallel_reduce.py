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
        x = layouts[0]
        nd = len(x.dim_axes)
        dims, keepdim, _ = _parse_dim_keepdim(extra_args, nd)
        op = _PARTIAL_OF.get(self.op_name, self.partial_op)
        # sum and mean are linear: a pending sum (or average) of the input stays pending on the result
        # -- e.g. the sum of a row-parallel product.  Every other reduction needs the reduced input.
        # (The reference's rule builds the result's layout afresh and loses the input's Partial status.)
        if op in ("sum", "avg") and all(p in (None, "sum", "avg") for p in x.partial):
            partial = list(x.partial)
        else:
            self._check_partial_inputs(layouts)
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
    """``max/min``: two tensors -> element-wise; full reduction -> Partial(max/min); with ``dim`` ->
    ``(values, indices)``.  Reducing a sharded dim leaves the values Partial(max/min) on its mesh axes,
    as the reference does (parallel_reduce.py:201-311 there); the indices are resolved on the spot --
    global positions of the first winning element, found with one max and one min all-reduce per mesh
    axis -- where the reference returns each rank's local positions."""

    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        x = layouts[0]
        if len(layouts) > 1 and layouts[1] is not None:
            from .parallel_elementwise import ElementWiseDistributedOp
            return ElementWiseDistributedOp._infer(self, layouts, extra_args)
        nd = len(x.dim_axes)
        dims, keepdim, given = _parse_dim_keepdim(extra_args, nd)
        op = "max" if "max" in self.op_name else "min"
        if not given:
            partial = [None] * x.mesh.ndim
            for axes in x.dim_axes:
                for a in axes:
                    partial[a] = op
            return make(x, [], partial)
        out_axes = [(() if d in dims else axes) for d, axes in enumerate(x.dim_axes) if keepdim or d not in dims]
        partial = [None] * x.mesh.ndim
        for d in dims:
            for a in x.dim_axes[d]:
                partial[a] = op
        return (make(x, out_axes, partial), make(x, out_axes))

    def get_expand_impl(self, func, output_layout, layouts, extra_args):
        x = layouts[0]
        if (len(layouts) > 1 and layouts[1] is not None) or not isinstance(output_layout, tuple):
            return None
        dims, _, _ = _parse_dim_keepdim(extra_args, len(x.dim_axes))
        axes = x.dim_axes[dims[0]]
        if not axes:
            return None
        import torch
        from ....collectives import cc
        mesh = x.mesh
        groups = [mesh.get_group(a) for a in axes]
        shard_idx = 0
        for a in axes:
            shard_idx = shard_idx * mesh.mesh_shape[a] + mesh.get_local_rank(a)
        is_max = "max" in self.op_name
        dim = dims[0]

        def impl(t, *a, **k):
            vals, idx = func(t, *a, **k)
            best = vals.detach().clone()
            for g in groups:
                cc.all_reduce_(best, "max" if is_max else "min", g)
            cand = torch.where(vals.detach() == best, idx + shard_idx * t.shape[dim],
                               torch.full_like(idx, torch.iinfo(idx.dtype).max))
            for g in groups:
                cc.all_reduce_(cand, "min", g)
            return vals, cand
        return impl


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
