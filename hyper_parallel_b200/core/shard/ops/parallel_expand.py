"""``expand`` / ``expand_as`` / ``broadcast_to`` / ``repeat``: a sharded dim cannot be expanded
(hyper_parallel/core/shard/ops/parallel_expand.py:22-246 of the reference).  Sizes are global;
the op runs with local sizes."""
from ._common import make, split_shapes
from .parallel_ops import DistributedOp
from .parallel_reshape import _flatten_shape_args


class ExpandDistributedOp(DistributedOp):
    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        x = layouts[0]
        extra, shapes = split_shapes(extra_args)
        in_shape = shapes[0]
        sizes = _flatten_shape_args(extra)
        off = len(sizes) - len(in_shape)
        if off < 0:
            raise ValueError(f"For {self.op_name}, target has fewer dims than the input")
        out_axes, local = [], []
        for d, s in enumerate(sizes):
            src = d - off
            if src < 0:
                out_axes.append(()); local.append(s)
                continue
            axes = x.dim_axes[src]
            if self.op_name == "repeat":
                if axes and s != 1:
                    raise ValueError(f"For repeat, sharded dim {src} cannot be repeated")
                out_axes.append(axes); local.append(s)
                continue
            if s in (-1, in_shape[src]):
                out_axes.append(axes)
                local.append(-1)
            else:
                if axes:
                    raise ValueError(f"For {self.op_name}, sharded dim {src} cannot be expanded")
                if in_shape[src] != 1:
                    raise ValueError(f"For {self.op_name}, dim {src} of size {in_shape[src]} cannot expand to {s}")
                out_axes.append(()); local.append(s)
        out = make(x, out_axes)
        out._local_sizes = tuple(local)
        return out

    def get_expand_impl(self, func, output_layout, layouts, extra_args):
        local = output_layout._local_sizes
        return lambda x, *a, **k: func(x, local)


class ExpandAsDistributedOp(DistributedOp):
    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        x, other = layouts[0], layouts[1]
        if other is None:
            raise ValueError("For expand_as, the target must be a distributed tensor")
        _, shapes = split_shapes(extra_args)
        in_shape, tgt_shape = shapes[0], shapes[1]
        off = len(tgt_shape) - len(in_shape)
        for d in range(len(in_shape)):
            if in_shape[d] != tgt_shape[d + off] and x.dim_axes[d]:
                raise ValueError(f"For expand_as, sharded dim {d} cannot be expanded")
            if in_shape[d] == tgt_shape[d + off] and x.dim_axes[d] != other.dim_axes[d + off]:
                raise ValueError("For expand_as, kept dims must be sharded like the target")
        return make(x, other.dim_axes)
