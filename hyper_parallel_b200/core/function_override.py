"""Module full-backward hooks on DTensor arguments.

``torch.utils.hooks.BackwardHook`` passes the tensor arguments of a module through
``torch.nn.modules._functions.BackwardHookFunction.apply`` and then looks for the resulting
``grad_fn`` on them.  ``Function.apply`` does not go through ``__torch_function__``, so with DTensor
arguments the node would be attached to the wrapper objects instead of the local tensors that carry
the autograd graph, and ``register_full_backward_hook`` / ``register_full_backward_pre_hook`` on a
module fed with DTensors would fail ("Error while setting up backward hooks").  The reference
replaces the function for the same reason
(hyper_parallel/platform/torch/function_override.py:24-79).  Here ``apply`` is wrapped: DTensors
are unwrapped, the original function runs on the local tensors, and the results are re-wrapped
with the layouts of the corresponding inputs.
"""
from __future__ import annotations

import torch
from torch.nn.modules import _functions

_ORIGINAL = _functions.BackwardHookFunction


class _DTensorAwareBackwardHookFunction:
    """Drop-in for ``BackwardHookFunction`` (only ``apply`` is used by torch)."""

    @staticmethod
    def apply(*args):
        from .dtensor import DTensor
        if not any(isinstance(a, DTensor) for a in args):
            return _ORIGINAL.apply(*args)
        local = [a.to_local() if isinstance(a, DTensor) else a for a in args]
        out = _ORIGINAL.apply(*local)
        return tuple(DTensor._wrap(o, a.layout) if isinstance(a, DTensor) else o for o, a in zip(out, args))


def install() -> None:
    if _functions.BackwardHookFunction is not _DTensorAwareBackwardHookFunction:
        _functions.BackwardHookFunction = _DTensorAwareBackwardHookFunction


def uninstall() -> None:
    _functions.BackwardHookFunction = _ORIGINAL
