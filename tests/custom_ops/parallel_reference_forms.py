"""Test-only rules written against the two special calling conventions of the reference's dispatcher
(``infer_layout_suffix: Reshape`` and ``Slice``): the rule gets ``[shape, global input shape]`` /
``[begin, end, global input shape]`` and returns the output layout together with the arguments the
local call needs."""
from hyper_parallel_b200 import DistributedOp


class FoldRowsDistributedOp(DistributedOp):
    """``fold_rows(x, shape)``: a reshape that keeps dim 0 (the only dim that may be sharded)."""

    def infer_layout(self, layouts, extra_args):
        x = layouts[0]
        shape, in_shape = extra_args
        if shape[0] != in_shape[0]:
            raise ValueError("fold_rows keeps dim 0")
        if any(a != "None" for a in x.alias_tensor_map[1:]):
            raise ValueError("fold_rows: only dim 0 may be sharded")
        out = x(x.alias_tensor_map[0], *(["None"] * (len(shape) - 1)))
        factor = x.mesh.mesh_shape[x.mesh.mesh_dim_names.index(x.alias_tensor_map[0])] \
            if x.alias_tensor_map[0] != "None" else 1
        return out, (shape[0] // factor,) + tuple(shape[1:])


class WindowDistributedOp(DistributedOp):
    """``window(x, begin, end)``: per-dim slice; a sharded dim must be taken whole and its bounds
    become those of the local shard."""

    def infer_layout(self, layouts, extra_args):
        x = layouts[0]
        begin, end, shape = extra_args
        new_begin, new_end = list(begin), list(end)
        for d, name in enumerate(x.alias_tensor_map):
            if name == "None":
                continue
            if begin[d] != 0 or end[d] != shape[d]:
                raise ValueError(f"window: sharded dim {d} must be taken whole")
            factor = x.mesh.mesh_shape[x.mesh.mesh_dim_names.index(name)]
            new_end[d] = shape[d] // factor
        return x(*x.alias_tensor_map), tuple(new_begin), tuple(new_end)
