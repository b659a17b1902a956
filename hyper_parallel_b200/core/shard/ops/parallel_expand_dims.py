"""``unsqueeze``: insert an unsharded dim, keep Partial
(hyper_parallel/core/shard/ops/parallel_expand_dims.py:22-74 of the reference)."""
from ._common import make
from .parallel_ops import DistributedOp


class ExpandDimsDistributedOp(DistributedOp):
    _allow_partial_inputs = True

    def infer_layout(self, layouts, extra_args):
        x = layouts[0]
        nd = len(x.dim_axes)
        dim = int(extra_args[0])
        if dim < 0:
            dim += nd + 1
        if not 0 <= dim <= nd:
            raise IndexError(f"For {self.op_name}, dim {extra_args[0]} out of range")
        axes = list(x.dim_axes)
        axes.insert(dim, ())
        return make(x, axes, x.partial)
