"""Activation recomputation with selective save / recompute / swap policies.

API of hyper_parallel/core/activation_checkpoint/activation_checkpoint.py:23-79 and the
selective-checkpoint dispatch modes of hyper_parallel/platform/torch/activation_checkpoint/sac.py
of the reference, implemented with two small ``TorchDispatchMode``s of our own:

* during the original forward, the output of every op whose policy is ``*_SAVE`` or ``MUST_SWAP``
  is cached (``MUST_SWAP``: moved to pinned host memory asynchronously);
* during recomputation those ops are not executed again: their cached outputs are replayed (swapped
  ones are copied back first); everything else is recomputed.
"""
from __future__ import annotations

import contextlib
import enum
from collections import defaultdict
from typing import Callable, Optional

import torch
from torch import nn
from torch.utils._python_dispatch import TorchDispatchMode
from torch.utils._pytree import tree_map
from torch.utils.checkpoint import checkpoint as _torch_checkpoint

from .swap import SwapTensor


class CheckpointPolicy(enum.Enum):
    MUST_SAVE = 0
    PREFER_SAVE = 1
    MUST_RECOMPUTE = 2
    PREFER_RECOMPUTE = 3
    MUST_SWAP = 4


_SAVE = (CheckpointPolicy.MUST_SAVE, CheckpointPolicy.PREFER_SAVE)


def _policy(policy_fn, func, args, kwargs) -> CheckpointPolicy:
    p = policy_fn(func, *args, **kwargs) if policy_fn is not None else CheckpointPolicy.PREFER_RECOMPUTE
    if isinstance(p, bool):
        return CheckpointPolicy.MUST_SAVE if p else CheckpointPolicy.PREFER_RECOMPUTE
    if not isinstance(p, CheckpointPolicy):
        # accept torch.utils.checkpoint.CheckpointPolicy members by name
        return CheckpointPolicy[p.name]
    return p


class _CachingMode(TorchDispatchMode):
    def __init__(self, policy_fn, storage):
        super().__init__()
        self.policy_fn, self.storage = policy_fn, storage

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        out = func(*args, **kwargs)
        pol = _policy(self.policy_fn, func, args, kwargs)
        if pol in _SAVE:
            self.storage[func].append(tree_map(lambda t: t.detach() if isinstance(t, torch.Tensor) else t, out))
        elif pol == CheckpointPolicy.MUST_SWAP:
            def swap(t):
                if not isinstance(t, torch.Tensor):
                    return t
                st = SwapTensor(t.detach())
                st.launch_offload()
                return st
            self.storage[func].append(tree_map(swap, out))
        return out


class _CachedMode(TorchDispatchMode):
    def __init__(self, policy_fn, storage):
        super().__init__()
        self.policy_fn, self.storage = policy_fn, storage

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        pol = _policy(self.policy_fn, func, args, kwargs)
        if pol in _SAVE or pol == CheckpointPolicy.MUST_SWAP:
            cached = self.storage.get(func)
            if not cached:
                raise RuntimeError(f"selective checkpoint: no cached output left for {func} -- the recomputed "
                                   "forward ran a different sequence of ops than the original one")
            out = cached.pop(0)
            return tree_map(lambda t: t.get() if isinstance(t, SwapTensor) else t, out)
        return func(*args, **kwargs)


def create_selective_checkpoint_contexts(policy_fn):
    storage = defaultdict(list)
    return _CachingMode(policy_fn, storage), _CachedMode(policy_fn, storage)


def checkpoint(function: Callable, *args, swap_inputs: bool = False, policy_fn: Optional[Callable] = None,
               **kwargs):
    """Run ``function(*args, **kwargs)`` without keeping its intermediate activations; they are
    recomputed in backward (non-reentrant).  ``policy_fn(op, *args, **kwargs) -> CheckpointPolicy``
    selects per op what is saved, recomputed or swapped to the host.  ``swap_inputs`` additionally
    keeps the tensor arguments on the host between forward and backward."""
    context_fn = (lambda: create_selective_checkpoint_contexts(policy_fn)) if policy_fn is not None \
        else (lambda: (contextlib.nullcontext(), contextlib.nullcontext()))
    if not swap_inputs:
        return _torch_checkpoint(function, *args, use_reentrant=False, context_fn=context_fn, **kwargs)

    # inputs go to the host right away and come back for the recomputation
    handles = []
    for a in args:
        if isinstance(a, torch.Tensor) and not isinstance(a, nn.Parameter) and a.numel() > 0:
            st = SwapTensor(a.detach())
            handles.append(st)
        else:
            handles.append(None)
    first = [True]

    def run(*inner):
        if first[0]:
            first[0] = False
            out = function(*inner, **kwargs)
            for st in handles:
                if st is not None:
                    st.launch_offload()
            return out
        reloaded = []
        for a, st in zip(inner, handles):
            if st is None:
                reloaded.append(a)
            else:
                t = st.get().detach().requires_grad_(a.requires_grad)
                # gradients must flow to the original argument: add a zero-cost dependency
                reloaded.append(t if not a.requires_grad else a + (t - a).detach())
        return function(*reloaded, **kwargs)

    return _torch_checkpoint(run, *args, use_reentrant=False, context_fn=context_fn)


class CheckpointWrapper(nn.Module):
    def __init__(self, module: nn.Module, policy_fn=None, swap_inputs: bool = False, checkpoint_fn=None,
                 **checkpoint_fn_kwargs):
        super().__init__()
        self._checkpoint_wrapped_module = module
        self.policy_fn, self.swap_inputs = policy_fn, swap_inputs
        self.checkpoint_fn, self.checkpoint_fn_kwargs = checkpoint_fn, checkpoint_fn_kwargs
        self._register_state_dict_hook(self._strip)
        self._register_load_state_dict_pre_hook(self._add)

    @staticmethod
    def _strip(module, state_dict, prefix, local_metadata):
        tag = prefix + "_checkpoint_wrapped_module."
        for k in list(state_dict.keys()):
            if k.startswith(tag):
                state_dict[prefix + k[len(tag):]] = state_dict.pop(k)
        return state_dict

    @staticmethod
    def _add(state_dict, prefix, *args):
        tag = prefix + "_checkpoint_wrapped_module."
        for k in list(state_dict.keys()):
            if k.startswith(prefix) and not k.startswith(tag):
                state_dict[tag + k[len(prefix):]] = state_dict.pop(k)

    def forward(self, *args, **kwargs):
        if self.checkpoint_fn is not None and self.checkpoint_fn is not checkpoint:
            # a checkpoint function of the caller's (e.g. torch.utils.checkpoint.checkpoint with its own
            # keyword arguments), as the reference's wrapper takes it
            return self.checkpoint_fn(self._checkpoint_wrapped_module, *args, **self.checkpoint_fn_kwargs, **kwargs)
        return checkpoint(self._checkpoint_wrapped_module, *args, swap_inputs=self.swap_inputs,
                          policy_fn=self.policy_fn, **kwargs)


def checkpoint_wrapper(module: nn.Module, policy_fn=None, swap_inputs: bool = False, *, checkpoint_fn=None,
                       **checkpoint_fn_kwargs) -> CheckpointWrapper:
    """Wrap ``module`` so that its forward runs under activation checkpointing.  Either this package's
    :func:`checkpoint` with ``policy_fn`` / ``swap_inputs``, or -- the reference's form
    (core/activation_checkpoint/activation_checkpoint.py:60-79 there) -- ``checkpoint_fn`` with the keyword
    arguments to hand to it."""
    return CheckpointWrapper(module, policy_fn, swap_inputs, checkpoint_fn, **checkpoint_fn_kwargs)
