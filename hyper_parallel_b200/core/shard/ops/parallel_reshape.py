"""Layout rule for ``reshape`` / ``view`` / ``flatten`` / ``unflatten``.

Capability of hyper_parallel/core/shard/ops/parallel_reshape.py:56-239 of the
reference: the target shape is given in **global** sizes (one ``-1`` allowed); the
rule matches groups of input dims to groups of output dims, moves the sharding of
a group to its leading output dim (only the leading dim of a merged group may be
sharded, and the receiving dim must stay divisible), and runs the op with the
derived **local** target shape.
"""
from __future__ import annotations

from typing import List, Sequence

from ._common import make, split_shapes
from .parallel_ops import DistributedOp


def _flatten_shape_args(args) -> List[int]:
    out: List[int] = []
    for a in args:
        if isinstance(a, (list, tuple)):
            out.extend(int(i) for i in a)
        elif isinstance(a, int) and not isinstance(a, bool):
            out.append(int(a))
    return out


def _resolve_minus_one(target: List[int], numel: int) -> List[int]:
    if target.count(-1) > 1:
        raise ValueError("only one dimension of the target shape may be -1")
    if -1 in target:
        known = 1
        for t in target:
            if t != -1:
                known *= t
        if known == 0 or numel % known:
            raise ValueError(f"shape {target} is invalid for input of size {numel}")
        target = [numel // known if t == -1 else t for t in target]
    return target


def infer_reshape(op_name, layout, in_shape: Sequence[int], target: Sequence[int]):
    """Returns (out_dim_axes, local_target_shape)."""
    numel = 1
    for s in in_shape:
        numel *= s
    target = _resolve_minus_one(list(target), numel)
    tn = 1
    for t in target:
        tn *= t
    if tn != numel:
        raise ValueError(f"For {op_name}, shape {tuple(target)} is invalid for input of size {numel}")
    out_axes: List[tuple] = [()] * len(target)
    i = j = 0
    ni, nj = len(in_shape), len(target)
    while i < ni or j < nj:
        # grow a group until the products match
        gi, gj = [i] if i < ni else [], [j] if j < nj else []
        pi = in_shape[i] if i < ni else 1
        pj = target[j] if j < nj else 1
        i += 1 if i < ni else 0
        j += 1 if j < nj else 0
        while pi != pj:
            if pi < pj:
                if i >= ni:
                    raise ValueError(f"For {op_name}, cannot match shapes {tuple(in_shape)} -> {tuple(target)}")
                pi *= in_shape[i]; gi.append(i); i += 1
            else:
                if j >= nj:
                    raise ValueError(f"For {op_name}, cannot match shapes {tuple(in_shape)} -> {tuple(target)}")
                pj *= target[j]; gj.append(j); j += 1
        # absorb trailing size-1 dims into the group boundaries lazily (handled by next iterations)
        sharded = [d for d in gi if layout.dim_axes[d]]
        if not sharded:
            continue
        # only the leading non-unit input dim of the group may be sharded
        lead_in = next((d for d in gi if in_shape[d] != 1), gi[0])
        if sharded != [lead_in]:
            raise ValueError(f"For {op_name}, only the leading dim of a merged/split group may be sharded "
                             f"(group dims {gi}, sharded {sharded})")
        axes = layout.dim_axes[lead_in]
        factor = 1
        for a in axes:
            factor *= layout.mesh_shape[a]
        lead_out = next((d for d in gj if target[d] != 1), gj[0])
        if target[lead_out] % factor:
            raise ValueError(f"For {op_name}, output dim {lead_out} of size {target[lead_out]} cannot "
                             f"carry a sharding factor of {factor}")
        out_axes[lead_out] = axes
    local = []
    for d, t in enumerate(target):
        f = 1
        for a in out_axes[d]:
            f *= layout.mesh_shape[a]
        local.append(t // f)
    return out_axes, local


class ReshapeDistributedOp(DistributedOp):
    _with_shape_convention = True     # called in the "WithShape" form although registered as "Reshape"

    def _target(self, extra, in_shape):
        if self.op_name == "flatten":
            ints = [a for a in extra if isinstance(a, int) and not isinstance(a, bool)]
            nd = len(in_shape)
            s = ints[0] if ints else 0
            e = ints[1] if len(ints) > 1 else -1
            s = s + nd if s < 0 else s
            e = e + nd if e < 0 else e
            merged = 1
            for v in in_shape[s:e + 1]:
                merged *= v
            return list(in_shape[:s]) + [merged] + list(in_shape[e + 1:])
        if self.op_name == "unflatten":
            dim = extra[0]
            nd = len(in_shape)
            dim = dim + nd if dim < 0 else dim
            sizes = _resolve_minus_one(list(extra[1]), in_shape[dim])
            return list(in_shape[:dim]) + sizes + list(in_shape[dim + 1:])
        return _flatten_shape_args(extra)

    def infer_layout(self, layouts, extra_args):
        x = layouts[0]
        if (len(extra_args) == 2 and all(isinstance(a, (tuple, list)) and a and all(isinstance(i, int) for i in a)
                                         for a in extra_args)):
            # the reference's "Reshape" form, for code that calls the rule directly:
            # (target shape, global input shape) -> (layout, local target shape)
            out_axes, local = infer_reshape(self.op_name, x, tuple(extra_args[1]), list(extra_args[0]))
            return make(x, out_axes, x.partial), list(local)
        extra, shapes = split_shapes(extra_args)
        in_shape = shapes[0]
        target = self._target(extra, in_shape)
        out_axes, local = infer_reshape(self.op_name, x, in_shape, target)
        out = make(x, out_axes, x.partial)
        out._local_target = tuple(local)
        return out

    def get_expand_impl(self, func, output_layout, layouts, extra_args):
        local = output_layout._local_target
        if self.op_name in ("flatten", "unflatten"):
            return lambda x, *a, **k: x.reshape(local)
        return lambda x, *a, **k: func(x, local)
