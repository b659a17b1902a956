"""``squeeze``: a removed dim must be an unsharded size-1 dim
(hyper_parallel/core/shard/ops/parallel_squeeze.py:22-231 of the reference)."""
from ._common import make, norm_dim, split_shapes
from .parallel_ops import DistributedOp


class SqueezeDistributedOp(DistributedOp):
    _allow_partial_inputs = True

    def infer_layout(self, layouts, extra_args):
        x = layouts[0]
        extra, shapes = split_shapes(extra_args)
        shape = shapes[0]
        nd = len(shape)
        if extra:
            dims = extra[0] if isinstance(extra[0], (list, tuple)) else [a for a in extra if isinstance(a, int)]
            dims = [norm_dim(d, nd) for d in dims]
        else:
            dims = [d for d in range(nd) if shape[d] == 1]
        out = []
        for d in range(nd):
            if d in dims and shape[d] == 1:
                if x.dim_axes[d]:
                    raise ValueError(f"For {self.op_name}, dim {d} is sharded and cannot be squeezed")
                continue
            out.append(x.dim_axes[d])
        return make(x, out, x.partial)
