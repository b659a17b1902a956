"""``embedding(indices, weight)``: out = indices map + weight[-1] map; the vocabulary dim of
the weight must be unsharded (hyper_parallel/core/shard/ops/parallel_embedding.py:23-82)."""
from ._common import make
from .parallel_ops import DistributedOp


class EmbeddingDistributedOp(DistributedOp):
    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        idx, w = layouts[0], layouts[1]
        if w is None:
            raise ValueError("For embedding, the weight must be a distributed tensor")
        if w.dim_axes[0]:
            raise ValueError("For embedding, the vocabulary dim of the weight must not be sharded")
        idx_axes = list(idx.dim_axes) if idx is not None else None
        if idx_axes is None:
            raise ValueError("For embedding, the indices must be a distributed tensor")
        used = {a for ax in idx_axes for a in ax}
        if used & set(w.dim_axes[1]):
            raise ValueError("For embedding, indices and the hidden dim share a mesh axis")
        return make(w, idx_axes + [w.dim_axes[1]])
