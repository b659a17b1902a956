"""``layer_norm`` / ``rms_norm``: the normalised (trailing) dims must be unsharded
(hyper_parallel/core/shard/ops/parallel_norm.py:22-169 of the reference)."""
from ._common import make, require_unsharded
from .parallel_ops import DistributedOp


class NormDistributedOp(DistributedOp):
    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        x = layouts[0]
        shape = next((a for a in extra_args if isinstance(a, (list, tuple))), None)
        n = len(shape) if shape is not None else 1
        nd = len(x.dim_axes)
        require_unsharded(self.op_name, x, range(nd - n, nd), "normalised")
        for l in layouts[1:]:
            if l is not None and any(l.dim_axes):
                raise ValueError(f"For {self.op_name}, weight/bias must be replicated")
        return make(x, x.dim_axes)


LayerNormDistributedOp = NormDistributedOp
