"""Per-module state and hook scheduling of ``fully_shard``.

Roles of hyper_parallel/core/fully_shard/hsdp_scheduler.py:32-194, hsdp_state.py:22-177 and
hyper_parallel/platform/torch/fully_shard/state.py:38-250, scheduler.py:25-129 of the reference:
forward-pre casts inputs and unshards (consuming a prefetch), forward-post reshards and casts
outputs, backward re-gathers, and each module's gradient reduce-scatters are launched
asynchronously in its post-backward and drained one module later (so the reduction of layer *i*
overlaps the backward of layer *i-1*) or by the end-of-backward callback.
"""
from __future__ import annotations

from typing import List

import torch
from torch import nn
from torch.autograd import Variable

from .param import FSDPParam
from .utils import MixedPrecisionPolicy

_PRE_REDUCE: List["FSDPState"] = []      # states whose reductions are in flight (FIFO)
_ALL_STATES: List["FSDPState"] = []
_ROOT_QUEUED = False


def _tree_map(obj, fn):
    if isinstance(obj, torch.Tensor):
        return fn(obj)
    if isinstance(obj, (list, tuple)):
        return type(obj)(_tree_map(o, fn) for o in obj)
    if isinstance(obj, dict):
        return {k: _tree_map(v, fn) for k, v in obj.items()}
    return obj


class _PostBackward(torch.autograd.Function):
    @staticmethod
    def forward(ctx, state, *inputs):
        ctx.state = state
        return inputs if len(inputs) > 1 else inputs[0]

    @staticmethod
    def backward(ctx, *grads):
        ctx.state.post_backward()
        return (None,) + grads


def _drain(keep_last: int = 0) -> None:
    while len(_PRE_REDUCE) > keep_last:
        st = _PRE_REDUCE.pop(0)
        for p in st.params:
            p.finish_reduce()


def _root_callback() -> None:
    global _ROOT_QUEUED
    _ROOT_QUEUED = False
    for st in _ALL_STATES:
        if st.in_backward or not st.is_sharded:
            st.post_backward(final=True)
    _drain(0)


class FSDPState:
    def __init__(self, module: nn.Module, params: List[FSDPParam], mp_policy: MixedPrecisionPolicy,
                 reshard_after_forward: bool):
        self.module = module
        self.params = params
        self.mp_policy = mp_policy
        self.reshard_after_forward = reshard_after_forward
        self.reshard_after_backward = True
        self.requires_gradient_sync = True
        self.requires_all_reduce = True
        self.is_last_backward = True
        self.reduce_op = "avg"
        self.fwd_prefetch: List[nn.Module] = []
        self.bwd_prefetch: List[nn.Module] = []
        self.is_sharded = True
        self.in_backward = False
        module.register_forward_pre_hook(self._pre_forward, with_kwargs=True)
        module.register_forward_hook(self._post_forward)
        _ALL_STATES.append(self)

    # ------------------------------------------------------------ (un)shard --
    def unshard(self, async_op: bool = False) -> None:
        for p in self.params:
            p.unshard(async_op=True)
        if not async_op:
            self.wait_for_unshard()

    def wait_for_unshard(self) -> None:
        for p in self.params:
            p.wait_for_unshard()
        self.is_sharded = False

    def reshard(self) -> None:
        for p in self.params:
            p.reshard()
        self.is_sharded = True

    @staticmethod
    def _prefetch(mods) -> None:
        for m in mods:
            st = getattr(m, "_fsdp_state", None)
            if st is not None and st.is_sharded:
                st.unshard(async_op=True)

    # ---------------------------------------------------------------- hooks --
    def _pre_forward(self, module, args, kwargs):
        self.unshard(async_op=True)
        self.wait_for_unshard()
        self._prefetch(self.fwd_prefetch)
        pd = self.mp_policy.param_dtype
        if pd is not None and self.mp_policy.cast_forward_inputs:
            cast = lambda t: t.to(pd) if t.is_floating_point() and t.dtype != pd else t  # noqa: E731
            args, kwargs = _tree_map(args, cast), _tree_map(kwargs, cast)
        if torch.is_grad_enabled():
            tensors = [a for a in args if isinstance(a, torch.Tensor) and a.requires_grad]
            if tensors:
                wrapped = _PostBackward.apply(self, *tensors)
                wrapped = wrapped if isinstance(wrapped, tuple) else (wrapped,)
                it = iter(wrapped)
                args = tuple(next(it) if (isinstance(a, torch.Tensor) and a.requires_grad) else a for a in args)
        return args, kwargs

    def _post_forward(self, module, args, output):
        if self.reshard_after_forward:
            self.reshard()
        if torch.is_grad_enabled():
            def reg(t):
                if t.requires_grad:
                    t.register_hook(self._pre_backward)
                return t
            _tree_map(output, reg)
        od = self.mp_policy.output_dtype
        if od is not None:
            output = _tree_map(output, lambda t: t.to(od) if t.is_floating_point() and t.dtype != od else t)
        return output

    def _pre_backward(self, grad):
        global _ROOT_QUEUED
        if not _ROOT_QUEUED:
            _ROOT_QUEUED = True
            Variable._execution_engine.queue_callback(_root_callback)
        if not self.in_backward:
            self.in_backward = True
            if self.is_sharded:
                self.unshard(async_op=True)
                self.wait_for_unshard()
            self._prefetch(self.bwd_prefetch)
        return grad

    def post_backward(self, final: bool = False) -> None:
        if not self.in_backward and not final:
            return
        self.in_backward = False
        if self.requires_gradient_sync:
            _drain(0)                         # reductions launched by the previous module
            launched = False
            for p in self.params:
                if p.unsharded_param.grad is not None:
                    p.reduce_grad(self.reduce_op, self.requires_all_reduce)
                    launched = True
            if launched:
                _PRE_REDUCE.append(self)
        if self.reshard_after_backward:
            self.reshard()


def reset_fully_shard_registry() -> None:
    _PRE_REDUCE.clear()
    _ALL_STATES.clear()
