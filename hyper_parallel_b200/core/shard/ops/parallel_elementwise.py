"""Layout rules for element-wise operators (unary, and broadcasting binary / ternary).

Behaviour follows hyper_parallel/core/shard/ops/parallel_elementwise.py:23-654 of
the reference: the output keeps the (broadcast-merged) sharding of the inputs; a
broadcast (size-1) dim may not be sharded; inputs with pending reductions are
rejected except by the ``...WithPartial`` rule (``mul``/``div``/``clone``/``neg``,
which are linear in their partial operand) and the ``Add`` rule (``add``/``sub``:
partial + partial keeps the status, partial + non-partial pre-divides the
non-partial operand by the number of partial ranks so that the later sum is right).
"""
from __future__ import annotations

from typing import List, Optional


from ._common import make, split_shapes
from .parallel_ops import DistributedOp


def _merge_broadcast(op_name, layouts, shapes):
    """Right-aligned broadcast merge of ``dim_axes``; returns (dim_axes, out_shape)."""
    tens = [(l, s) for l, s in zip(layouts, shapes or [None] * len(layouts)) if l is not None]
    plain = [s for l, s in zip(layouts, shapes or []) if l is None and s is not None]
    out_nd = max([len(l.dim_axes) for l, _ in tens] + [len(s) for s in plain])
    out_axes: List[tuple] = [()] * out_nd
    out_shape: List[int] = [1] * out_nd
    for l, s in tens:
        off = out_nd - len(l.dim_axes)
        for d, axes in enumerate(l.dim_axes):
            size = s[d] if s is not None else None
            od = d + off
            if size is not None:
                out_shape[od] = max(out_shape[od], size)
            if axes:
                if size == 1:
                    raise ValueError(f"For {op_name}, a broadcast (size-1) dim {d} must not be sharded")
                if out_axes[od] and out_axes[od] != axes:
                    raise ValueError(f"For {op_name}, inputs are sharded differently on dim {od}: "
                                     f"{out_axes[od]} vs {axes}")
                out_axes[od] = axes
    # every full-size distributed input must carry the merged sharding
    for l, s in tens:
        off = out_nd - len(l.dim_axes)
        for d, axes in enumerate(l.dim_axes):
            od = d + off
            if out_axes[od] and not axes and not (s is not None and s[d] == 1):
                raise ValueError(f"For {op_name}, dim {od} is sharded on one input but not on another; "
                                 "redistribute the inputs to a common layout first")
    for s in plain:
        off = out_nd - len(s)
        for d, size in enumerate(s):
            if out_axes[d + off] and size != 1:
                raise ValueError(f"For {op_name}, a plain tensor has full size on sharded dim {d + off}; "
                                 "wrap it in a DTensor with the matching layout")
    used = [a for axes in out_axes for a in axes]
    if len(used) != len(set(used)):
        raise ValueError(f"For {op_name}, a mesh axis would shard two output dims")
    return out_axes, out_shape


class ElementWiseDistributedOp(DistributedOp):
    """Unary or broadcasting n-ary element-wise op; no partial inputs."""

    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        return self._infer(layouts, extra_args)

    def _infer(self, layouts, extra_args, partial=None):
        _, shapes = split_shapes(extra_args)
        first = self.first_layout(layouts)
        n_t = sum(l is not None for l in layouts)
        if shapes is None or (n_t == 1 and all(s is None for l, s in zip(layouts, shapes) if l is None)):
            return make(first, first.dim_axes, partial if partial is not None else first.partial)
        axes, _ = _merge_broadcast(self.op_name, layouts, shapes)
        return make(first, axes, partial if partial is not None else [None] * first.mesh.ndim)


class ElementWiseWithPartialDistributedOp(ElementWiseDistributedOp):
    """Ops that are linear in one operand (``mul``, ``div``, ``clone``, ``neg``): Partial passes through."""

    _allow_partial_inputs = True

    def infer_layout(self, layouts, extra_args):
        partials = [l for l in layouts if l is not None and l.is_partial()]
        if len(partials) > 1:
            raise ValueError(f"For {self.op_name}, at most one input may have Partial status")
        partial = None
        if partials:
            p = partials[0]
            if any(op not in (None, "sum", "avg") for op in p.partial):
                raise ValueError(f"For {self.op_name}, only sum/avg Partial status can pass through")
            if self.op_name in ("div", "true_divide", "__truediv__", "div_") and layouts[0] is not p:
                raise ValueError(f"For {self.op_name}, the divisor must not be Partial")
            partial = list(p.partial)
            for l in layouts:
                if l is not None and l is not p:
                    for a, op in enumerate(partial):
                        if op is not None and a in l.sharded_axes:
                            raise ValueError(f"For {self.op_name}, mesh axis {a} is Partial on one input "
                                             "and shards another")
        return self._infer(layouts, extra_args, partial)


class AddDistributedOp(ElementWiseDistributedOp):
    """``add`` / ``sub``: keeps Partial; a non-partial operand is pre-divided by the partial ranks."""

    _allow_partial_inputs = True

    def infer_layout(self, layouts, extra_args):
        partial = self._merged_partial(layouts)
        return self._infer(layouts, extra_args, partial)

    def _merged_partial(self, layouts):
        tens = [l for l in layouts if l is not None]
        merged: List[Optional[str]] = [None] * tens[0].mesh.ndim
        for l in tens:
            for a, op in enumerate(l.partial):
                if op is None:
                    continue
                if op not in ("sum", "avg"):
                    raise ValueError(f"For {self.op_name}, only sum/avg Partial inputs are supported")
                if merged[a] is not None and merged[a] != op:
                    raise ValueError(f"For {self.op_name}, Partial ops differ on mesh axis {a}")
                merged[a] = op
        return merged

    def get_expand_impl(self, func, output_layout, layouts, extra_args):
        merged = output_layout.partial
        if not any(op == "sum" for op in merged):
            return None
        mesh = output_layout.mesh
        # scale factor for each positional operand that lacks a sum-partial axis of the result
        factors = []
        for l in layouts:
            f = 1
            for a, op in enumerate(merged):
                if op == "sum" and (l is None or l.partial[a] is None):
                    f *= mesh.mesh_shape[a]
            factors.append(f)
        if all(f == 1 for f in factors[:2]):
            return None
        inplace = self.op_name.endswith("_") or self.op_name.startswith("__i")
        if inplace and factors[0] != 1:
            raise ValueError(f"For {self.op_name}, an in-place update of a non-partial tensor with a "
                             "Partial operand is not defined")

        def impl(a, b, *rest, **kw):
            if factors[0] != 1:
                a = a / factors[0]
            if len(factors) > 1 and factors[1] != 1:
                b = b / factors[1]
            return func(a, b, *rest, **kw)
        return impl


class TupleElementWiseDistributedOp(DistributedOp):
    """Tuple pass-through: every output keeps the layout of the matching input."""

    _allow_partial_inputs = True

    def infer_layout(self, layouts, extra_args):
        return tuple(layouts)
