"""Saved-tensor hooks that swap activations to the host
(hyper_parallel/platform/torch/activation_checkpoint/activation_swap.py:54-192)."""
from __future__ import annotations

import enum
from typing import Callable, Optional

import torch
from torch import nn

from .swap import Storage, SwapManager, SwapTensor


class ActivationPolicy(enum.Enum):
    """What a ``policy_fn(tensor)`` may answer (reference activation_swap.py:35-38): keep the
    activation on the device, or swap it to the host.  A plain ``bool`` is accepted too
    (``True`` = swap)."""
    SAVE = 0
    SWAP = 1


def _wants_swap(answer) -> bool:
    return answer is ActivationPolicy.SWAP if isinstance(answer, ActivationPolicy) else bool(answer)


class AsyncSaveOnCpu(torch.autograd.graph.saved_tensors_hooks):
    """Inside this context every tensor saved for backward that ``policy_fn(tensor)`` accepts is
    replaced by a :class:`SwapTensor` whose device->host copy starts immediately (on a side
    stream) unless the tensor was registered with a :class:`SwapManager` group, in which case
    the manager's hooks decide when to copy."""

    def __init__(self, policy_fn: Optional[Callable[[torch.Tensor], bool]] = None, min_numel: int = 1024,
                 pin_memory: bool = True, managed: bool = False):
        mgr = SwapManager()

        def pack(t: torch.Tensor):
            if not isinstance(t, torch.Tensor) or t.numel() < min_numel or isinstance(t, nn.Parameter):
                return t
            if policy_fn is not None and not _wants_swap(policy_fn(t)):
                return t
            st = SwapTensor(t, pin_memory=pin_memory)
            if managed and mgr.current is not None:
                mgr.add_tensor(st)
            else:
                st.launch_offload()
            return Storage(st)

        def unpack(obj):
            if isinstance(obj, Storage):
                return obj.swap_tensor.take()
            return obj

        super().__init__(pack, unpack)


class SwapWrapper(nn.Module):
    """Runs the wrapped module under :class:`AsyncSaveOnCpu`; state-dict keys keep the inner names."""

    def __init__(self, module: nn.Module, policy_fn=None, managed: bool = True):
        super().__init__()
        self._swap_wrapped_module = module
        self._policy_fn = policy_fn
        self._managed = managed
        self._register_state_dict_hook(self._strip_prefix)
        self._register_load_state_dict_pre_hook(self._add_prefix)

    @staticmethod
    def _strip_prefix(module, state_dict, prefix, local_metadata):
        tag = prefix + "_swap_wrapped_module."
        for k in list(state_dict.keys()):
            if k.startswith(tag):
                state_dict[prefix + k[len(tag):]] = state_dict.pop(k)
        return state_dict

    @staticmethod
    def _add_prefix(state_dict, prefix, *args):
        tag = prefix + "_swap_wrapped_module."
        for k in list(state_dict.keys()):
            if k.startswith(prefix) and not k.startswith(tag):
                state_dict[tag + k[len(prefix):]] = state_dict.pop(k)

    def forward(self, *args, **kwargs):
        mgr = SwapManager()
        prev = mgr.current
        if self._managed and prev is None:
            mgr.current = self
            mgr.group_of(self).clear()
        try:
            with AsyncSaveOnCpu(self._policy_fn, managed=self._managed):
                return self._swap_wrapped_module(*args, **kwargs)
        finally:
            if self._managed and prev is None:
                mgr.current = None
                mgr.group_of(self).launch_offload()


def swap_wrapper(module: nn.Module, policy_fn=None) -> SwapWrapper:
    return SwapWrapper(module, policy_fn)
