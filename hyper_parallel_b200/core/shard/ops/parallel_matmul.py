"""Layout rules for ``matmul`` / ``mm`` / ``bmm`` / ``linear``.

Same rule as hyper_parallel/core/shard/ops/parallel_matmul.py:22-429 of the
reference: output = batch dims (broadcast-merged) + x[-2] + w[-1]; the contracting
dims of both operands must be sharded identically; a sharded contracting dim
makes the output ``Partial(sum)`` on those mesh axes.  No communication happens
here -- the all-reduce / reduce-scatter is issued later by ``reduce_partial`` or
``redistribute``.  ``linear`` takes the weight as ``[out, in]`` and, when the
contraction is sharded, divides the bias by the number of partial ranks so that
the later sum adds it exactly once.
"""
from __future__ import annotations

from ._common import make
from .parallel_ops import DistributedOp


def _merge_batch(op_name, xa, wa):
    n = max(len(xa), len(wa))
    xa = [()] * (n - len(xa)) + list(xa)
    wa = [()] * (n - len(wa)) + list(wa)
    out = []
    for a, b in zip(xa, wa):
        if a and b and a != b:
            raise ValueError(f"For {op_name}, batch dims are sharded differently: {a} vs {b}")
        out.append(a or b)
    return out


def _matmul_layout(op_name, x, w, w_is_out_in=False):
    """x: [..., m, k]; w: [..., k, n] (or [n, k] when ``w_is_out_in``)."""
    xa, wa = list(x.dim_axes), list(w.dim_axes)
    x_vec = len(xa) == 1
    w_vec = len(wa) == 1
    if x_vec:
        xa = [()] + xa
    if w_vec:
        wa = wa + [()] if not w_is_out_in else [()] + wa
    if w_is_out_in:
        w_n, w_k = wa[-2], wa[-1]
    else:
        w_k, w_n = wa[-2], wa[-1]
    x_k = xa[-1]
    if x_k != w_k:
        raise ValueError(f"For {op_name}, the contracting dims must be sharded identically, but got "
                         f"{x_k} (input) and {w_k} (weight)")
    batch = _merge_batch(op_name, xa[:-2], wa[:-2])
    out_axes = batch + [xa[-2], w_n]
    if x_vec:
        out_axes.pop(-2)
    if w_vec and not w_is_out_in:
        out_axes.pop(-1)
    used = [a for axes in out_axes for a in axes]
    if len(used) != len(set(used)):
        raise ValueError(f"For {op_name}, a mesh axis shards both operands' free dims: {out_axes}")
    partial = [None] * x.mesh.ndim
    for a in x_k:
        if a in used:
            raise ValueError(f"For {op_name}, mesh axis {a} shards both a free and a contracting dim")
        partial[a] = "sum"
    return make(x, out_axes, partial)


def _native_ok(*tensors) -> bool:
    """Local operands that the hand-written tcgen05 GEMM takes: CUDA, bf16."""
    import torch
    return all(isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == torch.bfloat16 for t in tensors)


class MatMulExtDistributedOp(DistributedOp):
    """``torch.matmul`` / ``mm`` / ``bmm`` / ``@``."""

    def get_expand_impl(self, func, output_layout, layouts, extra_args):
        # the local product of two DTensors runs on this library's tcgen05 GEMM (forward, dgrad and
        # wgrad) whenever the shards are bf16 CUDA matrices; anything else keeps the framework call
        def impl(x, w, *args, **kwargs):
            if not args and not kwargs and _native_ok(x, w) and w.dim() == 2 and x.dim() >= 2 and w.is_contiguous():
                from ....ops import functional as Fn
                return Fn.matmul(x, w)
            return func(x, w, *args, **kwargs)
        return impl

    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        tens = [l for l in layouts if l is not None]
        if len(tens) != 2 or layouts[0] is None or layouts[1] is None:
            raise ValueError(f"For {self.op_name}, both operands must be distributed tensors")
        return _matmul_layout(self.op_name, layouts[0], layouts[1])


MatMulDistributedOp = MatMulExtDistributedOp
BatchMatMulExtDistributedOp = MatMulExtDistributedOp
BatchMatMulDistributedOp = MatMulExtDistributedOp


class LinearDistributedOp(DistributedOp):
    """``F.linear(x, w[out, in], bias)``."""

    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        if layouts[0] is None or len(layouts) < 2 or layouts[1] is None:
            raise ValueError(f"For {self.op_name}, input and weight must be distributed tensors")
        out = _matmul_layout(self.op_name, layouts[0], layouts[1], w_is_out_in=True)
        bias = layouts[2] if len(layouts) > 2 else None
        if bias is not None and bias.dim_axes[-1] != out.dim_axes[-1]:
            raise ValueError(f"For {self.op_name}, the bias must be sharded like the output feature dim")
        return out

    def get_expand_impl(self, func, output_layout, layouts, extra_args):
        n = 1
        if output_layout.is_partial():
            for a, op in enumerate(output_layout.partial):
                if op is not None:
                    n *= output_layout.mesh.mesh_shape[a]

        def impl(x, w, bias=None):
            b = bias if (bias is None or n == 1) else bias / n
            if _native_ok(x, w) and w.dim() == 2:
                # the local product runs on this library's tcgen05 GEMM (forward, dgrad and wgrad)
                from ....ops import functional as Fn
                return Fn.linear(x, w, b)
            return func(x, w, b)
        return impl
