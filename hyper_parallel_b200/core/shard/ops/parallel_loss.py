"""Loss functions on distributed tensors: ``mse_loss`` / ``l1_loss`` (element-wise + reduction)
and ``cross_entropy`` / ``nll_loss`` (class dim unsharded).  A ``mean``/``sum`` reduction over
sharded dims leaves a pending ``avg``/``sum`` reduction, exactly like ``mean``/``sum``."""
from ._common import make, require_unsharded, split_shapes
from .parallel_ops import DistributedOp


def _reduction(extra):
    for a in extra:
        if isinstance(a, str) and a in ("mean", "sum", "none"):
            return a
    return "mean"


class ElementwiseLossDistributedOp(DistributedOp):
    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        x, y = layouts[0], layouts[1]
        if x is None or y is None or x.dim_axes != y.dim_axes:
            raise ValueError(f"For {self.op_name}, input and target must share one layout")
        extra, _ = split_shapes(extra_args)
        red = _reduction(extra)
        if red == "none":
            return make(x, x.dim_axes)
        partial = [None] * x.mesh.ndim
        for a in x.sharded_axes:
            partial[a] = "avg" if red == "mean" else "sum"
        return make(x, [], partial)


class CrossEntropyDistributedOp(DistributedOp):
    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        x, t = layouts[0], layouts[1]
        nd = len(x.dim_axes)
        cdim = 1 if nd > 1 else 0
        require_unsharded(self.op_name, x, [cdim], "class")
        batch_axes = [a for d, a in enumerate(x.dim_axes) if d != cdim]
        if t is not None and list(t.dim_axes) != batch_axes:
            raise ValueError(f"For {self.op_name}, the target must be sharded like the input batch dims")
        extra, _ = split_shapes(extra_args)
        red = _reduction(extra)
        if red == "none":
            return make(x, batch_axes)
        partial = [None] * x.mesh.ndim
        for a in x.sharded_axes:
            partial[a] = "avg" if red == "mean" else "sum"
        return make(x, [], partial)
