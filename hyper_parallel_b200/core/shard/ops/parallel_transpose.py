"""``transpose`` / ``permute`` / ``t`` / ``swapaxes`` / ``movedim``: permute the sharding map
(hyper_parallel/core/shard/ops/parallel_transpose.py:23-106 of the reference)."""
from __future__ import annotations

from ._common import make, norm_dim
from .parallel_ops import DistributedOp


class TransposeDistributedOp(DistributedOp):
    _allow_partial_inputs = True

    def infer_layout(self, layouts, extra_args):
        x = layouts[0]
        nd = len(x.dim_axes)
        axes = list(x.dim_axes)
        name = self.op_name
        if name in ("t", "T", "mT", "adjoint"):
            if nd < 2:
                return x
            perm = list(range(nd))
            perm[-1], perm[-2] = perm[-2], perm[-1]
        elif name in ("transpose", "swapaxes", "swapdims", "transpose_"):
            d0, d1 = norm_dim(extra_args[0], nd), norm_dim(extra_args[1], nd)
            perm = list(range(nd))
            perm[d0], perm[d1] = perm[d1], perm[d0]
        elif name == "movedim":
            src, dst = norm_dim(extra_args[0], nd), norm_dim(extra_args[1], nd)
            perm = [d for d in range(nd) if d != src]
            perm.insert(dst, src)
        else:  # permute
            dims = extra_args[0] if len(extra_args) == 1 and isinstance(extra_args[0], (list, tuple)) \
                else [a for a in extra_args if isinstance(a, int)]
            perm = [norm_dim(d, nd) for d in dims]
            if sorted(perm) != list(range(nd)):
                raise ValueError(f"For {name}, {dims} is not a permutation of {nd} dims")
        return make(x, [axes[p] for p in perm], x.partial)
