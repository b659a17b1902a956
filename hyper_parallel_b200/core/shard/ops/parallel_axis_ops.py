"""Rules for operators that work *along one axis*: that axis must be unsharded and the
output keeps the input's sharding map.

Covers the reference's ``softmax`` (parallel_activation_with_axis.py:21), ``cumsum``
(parallel_cumsum.py:22), ``sort`` (parallel_sort.py:22), ``topk`` (parallel_topk.py:21),
``repeat_interleave`` (parallel_repeat_interleave.py:22), ``index_select`` / ``gather``
(parallel_gather.py:23-147), ``scatter`` (parallel_scatter.py:22), ``unbind``
(parallel_unbind.py:23), ``split`` (parallel_split.py:23-210), ``cat`` (parallel_concat.py:23),
``pad`` (parallel_pad.py:22), ``isin`` (parallel_isin.py:22), ``multinomial``
(parallel_multinomial.py:23), ``masked_scatter`` (parallel_masked_scatter.py:22).
"""
from __future__ import annotations

from ._common import make, norm_dim, require_unsharded, split_shapes
from .parallel_ops import DistributedOp


def _first_int(extra, default=None):
    for a in extra:
        if isinstance(a, int) and not isinstance(a, bool):
            return a
    return default


class ActivationWithAxisDistributedOp(DistributedOp):
    """softmax / log_softmax / glu-like: ``dim`` (default -1) unsharded; layout unchanged."""

    default_dim = -1

    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        x = layouts[0]
        extra, _ = split_shapes(extra_args)
        nd = len(x.dim_axes)
        dim = norm_dim(_first_int(extra, self.default_dim), nd)
        require_unsharded(self.op_name, x, [dim], "operating")
        return make(x, x.dim_axes)


class CumsumDistributedOp(ActivationWithAxisDistributedOp):
    pass


class SortDistributedOp(ActivationWithAxisDistributedOp):
    """sort / argsort / topk-like ops returning (values, indices) or a single tensor."""

    def infer_layout(self, layouts, extra_args):
        lay = super().infer_layout(layouts, extra_args)
        if self.op_name in ("argsort",):
            return lay
        return (lay, lay)


class TopKDistributedOp(DistributedOp):
    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        x = layouts[0]
        nd = len(x.dim_axes)
        ints = [a for a in extra_args if isinstance(a, int) and not isinstance(a, bool)]
        dim = norm_dim(ints[1] if len(ints) > 1 else -1, nd)
        require_unsharded(self.op_name, x, [dim], "top-k")
        lay = make(x, x.dim_axes)
        return (lay, lay)


class RepeatInterleaveDistributedOp(DistributedOp):
    """``repeat_interleave(x, repeats, dim=None)``; ``repeats`` an int or a (plain) tensor.  With a
    ``dim`` that dim must be unsharded and the layout is kept.  Without one the input is flattened:
    a sharding of dim 0 alone survives as the sharding of the flat result when every element repeats
    equally often (each rank's rows are one contiguous run of the flat tensor); any other sharding
    is refused."""

    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        x = layouts[0]
        nd = len(x.dim_axes)
        rest = [a for a in extra_args if not isinstance(a, bool) and a is not None]
        repeats = rest[0] if rest else None
        dim = next((a for a in rest[1:] if isinstance(a, int)), None)
        if dim is None:
            require_unsharded(self.op_name, x, range(1, nd), "flattened")
            if x.dim_axes[0] and not isinstance(repeats, int):
                require_unsharded(self.op_name, x, [0], "flattened")
            return make(x, [x.dim_axes[0] if nd else ()])
        dim = norm_dim(dim, nd)
        require_unsharded(self.op_name, x, [dim], "repeated")
        return make(x, x.dim_axes)


class IndexSelectDistributedOp(DistributedOp):
    """index_select(x, dim, index): ``dim`` unsharded; a distributed index must be replicated."""

    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        x = layouts[0]
        dim = norm_dim(_first_int(extra_args, 0), len(x.dim_axes))
        require_unsharded(self.op_name, x, [dim], "selected")
        for l in layouts[1:]:
            if l is not None and any(l.dim_axes):
                raise ValueError(f"For {self.op_name}, the index must be replicated")
        return make(x, x.dim_axes)


class GatherDistributedOp(DistributedOp):
    """gather(x, dim, index): ``dim`` unsharded; index sharded like x on the other dims."""

    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        x = layouts[0]
        dim = norm_dim(_first_int(extra_args, 0), len(x.dim_axes))
        require_unsharded(self.op_name, x, [dim], "gathered")
        idx = next((l for l in layouts[1:] if l is not None), None)
        if idx is not None:
            if idx.dim_axes != x.dim_axes:
                raise ValueError(f"For {self.op_name}, index must be sharded like the input")
            return make(x, idx.dim_axes)
        if any(x.dim_axes):
            raise ValueError(f"For {self.op_name}, a plain index needs a replicated input")
        return make(x, x.dim_axes)


GatherNdDistributedOp = GatherDistributedOp


class ScatterDistributedOp(DistributedOp):
    """scatter / scatter_add / scatter_: ``dim`` unsharded; index and src sharded like the input."""

    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        x = layouts[0]
        dim = norm_dim(_first_int(extra_args, 0), len(x.dim_axes))
        require_unsharded(self.op_name, x, [dim], "scatter")
        for what, l in zip(("Index", "Src"), [l for l in layouts[1:] if l is not None]):
            if l.dim_axes != x.dim_axes:
                raise ValueError(f"For {self.op_name}, index/src must be sharded like the input: {what} tensor "
                                 f"layout {l.alias_tensor_map} must match input layout {x.alias_tensor_map}")
        return make(x, x.dim_axes)


ScatterUpdateDistributedOp = ScatterDistributedOp


class MaskedScatterDistributedOp(DistributedOp):
    """masked_scatter consumes ``source`` in global element order: everything replicated."""

    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        for what, l in zip(("input", "mask", "source"), layouts):
            if l is not None and any(l.dim_axes):
                raise ValueError(f"For {self.op_name}, all inputs must be replicated, but {what} is sharded "
                                 f"({l.alias_tensor_map})")
        x = layouts[0]
        return make(x, x.dim_axes)


class UnbindDistributedOp(DistributedOp):
    def infer_layout(self, layouts, extra_args):
        x = layouts[0]
        extra, shapes = split_shapes(extra_args)
        nd = len(x.dim_axes)
        dim = norm_dim(_first_int(extra, 0), nd)
        require_unsharded(self.op_name, x, [dim], "unbound")
        lay = make(x, [a for d, a in enumerate(x.dim_axes) if d != dim], x.partial)
        return tuple([lay] * shapes[0][dim])

    _allow_partial_inputs = True


class SplitDistributedOp(DistributedOp):
    """split / chunk / tensor_split: split axis unsharded; every piece keeps the layout."""

    _allow_partial_inputs = True

    def infer_layout(self, layouts, extra_args):
        x = layouts[0]
        extra, shapes = split_shapes(extra_args)
        nd = len(x.dim_axes)
        size = shapes[0]
        spec = extra[0]
        dim = 0
        rest = [a for a in extra[1:] if isinstance(a, int) and not isinstance(a, bool)]
        if rest:
            dim = rest[0]
        dim = norm_dim(dim, nd)
        require_unsharded(self.op_name, x, [dim], "split")
        n = size[dim]
        if self.op_name == "chunk":
            per = -(-n // int(spec))
            count = -(-n // per) if per else 0
        elif isinstance(spec, (list, tuple)):
            count = len(spec) + (1 if self.op_name == "tensor_split" else 0)
        elif self.op_name == "tensor_split":
            count = int(spec)
        else:
            count = -(-n // int(spec))
        lay = make(x, x.dim_axes, x.partial)
        return tuple([lay] * count)


SplitWithSizeDistributedOp = SplitDistributedOp
SplitTensorDistributedOp = SplitDistributedOp


class ConcatDistributedOp(DistributedOp):
    """cat / concat (``WithTupleExpand``): identical maps, concat axis unsharded."""

    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        tens = [l for l in layouts if l is not None]
        if len(tens) != len(layouts):
            raise ValueError(f"For {self.op_name}, every input must be a distributed tensor")
        x = tens[0]
        extra, _ = split_shapes(extra_args)
        dim = norm_dim(_first_int(extra, 0), len(x.dim_axes))
        for l in tens:
            if l.dim_axes != x.dim_axes:
                raise ValueError(f"For {self.op_name}, inputs must share one sharding map")
        require_unsharded(self.op_name, x, [dim], "concat")
        return make(x, x.dim_axes)


class StackDistributedOp(DistributedOp):
    """stack (``WithTupleExpand``): identical maps; a new unsharded dim is inserted."""

    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        tens = [l for l in layouts if l is not None]
        x = tens[0]
        extra, _ = split_shapes(extra_args)
        nd = len(x.dim_axes)
        dim = _first_int(extra, 0)
        if dim < 0:
            dim += nd + 1
        for l in tens:
            if l.dim_axes != x.dim_axes:
                raise ValueError(f"For {self.op_name}, inputs must share one sharding map")
        axes = list(x.dim_axes)
        axes.insert(dim, ())
        return make(x, axes)


class PadDistributedOp(DistributedOp):
    """F.pad(x, pad): padded dims (counted from the last) must be unsharded."""

    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        x = layouts[0]
        pad = next((a for a in extra_args if isinstance(a, (list, tuple))), ())
        nd = len(x.dim_axes)
        dims = [nd - 1 - i for i in range(len(pad) // 2) if pad[2 * i] or pad[2 * i + 1]]
        require_unsharded(self.op_name, x, dims, "padded")
        return make(x, x.dim_axes)


class IsinDistributedOp(DistributedOp):
    """isin(elements, test_elements): output like ``elements``; test set replicated."""

    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        x = layouts[0]
        if x is None:
            raise ValueError("For isin, elements must be a distributed tensor")
        for l in layouts[1:]:
            if l is not None and any(l.dim_axes):
                raise ValueError("For isin, 'test_elements' must be unsharded (replicated), got "
                                 f"{l.alias_tensor_map}")
        return make(x, x.dim_axes)


class MultinomialDistributedOp(DistributedOp):
    """multinomial(probs[..., C], n): the category dim must be unsharded."""

    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        x = layouts[0]
        require_unsharded(self.op_name, x, [len(x.dim_axes) - 1], "category")
        return make(x, x.dim_axes)


class NewOnesDistributedOp(DistributedOp):
    """new_ones / new_zeros / new_full / new_empty(size): result is replicated."""

    _allow_partial_inputs = True

    def infer_layout(self, layouts, extra_args):
        x = layouts[0]
        size = next((a for a in extra_args if isinstance(a, (list, tuple))), None)
        if size is None:
            size = [a for a in extra_args if isinstance(a, int) and not isinstance(a, bool)]
        return make(x, [()] * len(size))


class LikeDistributedOp(DistributedOp):
    """zeros_like / ones_like / empty_like / full_like / rand_like: same sharding, no Partial."""

    _allow_partial_inputs = True

    def infer_layout(self, layouts, extra_args):
        x = layouts[0]
        return make(x, x.dim_axes)


def _in_rng_region(func, layout):
    """``func`` run inside the distributed RNG tracker's region for ``layout``: distinct shards draw
    from distinct Philox windows, replicas of a shard draw the same numbers, and every rank's
    tracker advances by the same amount -- whatever the ranks' local generators hold."""
    def impl(t, *a, **k):
        from ...random import get_rng_tracker
        with get_rng_tracker()._distribute_region(layout, tuple(t.shape)):
            return func(t, *a, **k)
    return impl


class RandomLikeDistributedOp(LikeDistributedOp):
    """rand_like / randn_like on a DTensor: the sharding of the input, values from the distributed
    RNG tracker (core/random.py).  The reference ships the tracker (hyper_parallel/core/random.py:
    123-296) but draws these from each rank's local generator, so ranks seeded alike give every
    shard the same numbers and ranks seeded differently let replicas diverge."""

    def get_expand_impl(self, func, output_layout, layouts, extra_args):
        return _in_rng_region(func, output_layout)


class DropoutDistributedOp(DistributedOp):
    """dropout / bernoulli: element-wise in the layout of the input, mask drawn in the tracker's region."""

    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        x = layouts[0]
        return make(x, x.dim_axes)

    def get_expand_impl(self, func, output_layout, layouts, extra_args):
        return _in_rng_region(func, output_layout)


class TrilDistributedOp(DistributedOp):
    """tril / triu: the last two dims must be unsharded."""

    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        x = layouts[0]
        nd = len(x.dim_axes)
        require_unsharded(self.op_name, x, [nd - 2, nd - 1], "matrix")
        return make(x, x.dim_axes)


class OneHotExtDistributedOp(DistributedOp):
    """F.one_hot(x, num_classes): appends an unsharded class dim.  With ``num_classes=-1`` the class
    count is the global maximum + 1, found with a max all-reduce over the sharded axes
    (hyper_parallel/core/shard/ops/parallel_one_hot_ext.py:75-129 of the reference)."""

    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        x = layouts[0]
        return make(x, list(x.dim_axes) + [()])

    def get_expand_impl(self, func, output_layout, layouts, extra_args):
        ints = [a for a in extra_args if isinstance(a, int) and not isinstance(a, bool)]
        num_classes = ints[0] if ints else -1
        x = layouts[0]
        if num_classes != -1 or not x.sharded_axes:
            return None
        from ....collectives import cc
        groups = [x.mesh.get_group(a) for a in sorted(x.sharded_axes)]

        def impl(t, *a, **k):
            m = t.max().reshape(1).clone()
            for g in groups:
                cc.all_reduce_(m, "max", g)
            return func(t, int(m.item()) + 1)
        return impl
