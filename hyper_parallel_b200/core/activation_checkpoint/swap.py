"""Activation swap (offload to pinned host memory and prefetch back).

Capability of hyper_parallel/core/activation_checkpoint/swap.py:30-465 of the reference:

* ``SwapTensor``: a device tensor with a pinned-CPU mirror and the state machine
  ``device -> d2h -> host -> h2d -> device``; copies run on a dedicated copy stream and are
  ordered against the compute stream with events;
* ``SwapGroup``: the swap tensors of one layer;
* ``SwapManager``: singleton holding groups by layer; ``set_forward_prefetch_layer(l_i, l_next)``
  installs hooks so that, in forward, finishing ``l_i`` launches its offload and waits for the
  offload of the layer before it, and, in backward, entering ``l_next`` launches the load of
  ``l_i``'s activations while ``l_next``'s own backward runs.

On CPU tensors everything degenerates to keeping the tensor (state transitions still happen),
which is what the CPU tests exercise.
"""
from __future__ import annotations

import enum
from typing import Dict, List, Optional

import torch


class SwapState(enum.Enum):
    DEVICE = "device"
    D2H = "d2h"
    HOST = "host"
    H2D = "h2d"


_COPY_STREAMS: Dict[int, "torch.cuda.Stream"] = {}


def copy_stream(device: torch.device):
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _COPY_STREAMS:
        _COPY_STREAMS[idx] = torch.cuda.Stream(device=idx)
    return _COPY_STREAMS[idx]


class Storage:
    """Holder that the saved-tensor hooks put into the autograd graph instead of the tensor."""

    __slots__ = ("swap_tensor",)

    def __init__(self, swap_tensor: "SwapTensor"):
        self.swap_tensor = swap_tensor


class SwapTensor:
    def __init__(self, tensor: torch.Tensor, pin_memory: bool = True):
        self.device = tensor.device
        self.shape, self.dtype = tensor.shape, tensor.dtype
        self.requires_grad = tensor.requires_grad
        self._device_tensor: Optional[torch.Tensor] = tensor
        self._host_tensor: Optional[torch.Tensor] = None
        self._event = None
        self.state = SwapState.DEVICE
        self.is_cuda = tensor.is_cuda
        self.pin_memory = pin_memory and self.is_cuda

    # --------------------------------------------------------------- offload --
    def launch_offload(self) -> None:
        """Start the device->host copy (asynchronous on CUDA)."""
        if self.state != SwapState.DEVICE:
            return
        t = self._device_tensor
        if not self.is_cuda:
            self._host_tensor = t
            self.state = SwapState.D2H
            return
        cs = copy_stream(self.device)
        cs.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(cs):
            host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=self.pin_memory)
            host.copy_(t, non_blocking=True)
            t.record_stream(cs)
            self._event = torch.cuda.Event()
            self._event.record(cs)
        self._host_tensor = host
        self.state = SwapState.D2H

    def wait_offload(self) -> None:
        """Make sure the copy is done, then drop the device copy."""
        if self.state != SwapState.D2H:
            return
        if self._event is not None:
            self._event.synchronize()
            self._event = None
        self._device_tensor = None
        self.state = SwapState.HOST

    # ------------------------------------------------------------------ load --
    def launch_load(self) -> None:
        if self.state == SwapState.D2H:
            self.wait_offload()
        if self.state != SwapState.HOST:
            return
        if not self.is_cuda:
            self._device_tensor = self._host_tensor
            self.state = SwapState.H2D
            return
        cs = copy_stream(self.device)
        with torch.cuda.stream(cs):
            dev = torch.empty(self.shape, dtype=self.dtype, device=self.device)
            dev.copy_(self._host_tensor, non_blocking=True)
            self._event = torch.cuda.Event()
            self._event.record(cs)
        self._device_tensor = dev
        self.state = SwapState.H2D

    def wait_load(self, keep_host: bool = False) -> torch.Tensor:
        if self.state in (SwapState.HOST, SwapState.D2H):
            self.launch_load()
        if self.state == SwapState.H2D:
            if self._event is not None:
                cur = torch.cuda.current_stream(self.device)
                cur.wait_event(self._event)
                self._device_tensor.record_stream(cur)      # allocated on the copy stream, read on this one
                self._event = None
            if not keep_host:
                self._host_tensor = None
            self.state = SwapState.DEVICE
        return self._device_tensor

    def get(self) -> torch.Tensor:
        return self.wait_load()

    def take(self) -> torch.Tensor:
        """The device tensor for one use by autograd.  When a host copy exists this object lets go of
        the device copy afterwards, so the memory returns to the allocator as soon as the backward
        node that asked for it is done; a later request loads from the host copy again."""
        t = self.wait_load(keep_host=True)
        if self._host_tensor is not None and self.is_cuda:
            self._device_tensor = None
            self.state = SwapState.HOST
        return t


# the reference's method names (core/activation_checkpoint/swap.py:51-131 there)
SwapTensor.async_offload = SwapTensor.launch_offload
SwapTensor.async_load = SwapTensor.launch_load
SwapTensor.get_val = SwapTensor.get


class SwapGroup:
    """The swap tensors that belong to one layer."""

    def __init__(self, name: str = ""):
        self.name = name
        self.tensors: List[SwapTensor] = []

    def add(self, st: SwapTensor) -> None:
        self.tensors.append(st)

    def launch_offload(self) -> None:
        for t in self.tensors:
            t.launch_offload()

    def wait_offload(self) -> None:
        for t in self.tensors:
            t.wait_offload()

    def launch_load(self) -> None:
        for t in self.tensors:
            t.launch_load()

    def wait_load(self) -> None:
        for t in self.tensors:
            t.wait_load(keep_host=True)

    def clear(self) -> None:
        self.tensors = []


class SwapManager:
    """Process-wide registry of swap groups keyed by layer (singleton)."""

    _instance: Optional["SwapManager"] = None

    def __new__(cls):
        if cls._instance is None:
            cls._instance = super().__new__(cls)
            cls._instance.groups = {}
            cls._instance.current = None
            cls._instance._prev_of = {}
        return cls._instance

    def group_of(self, layer) -> SwapGroup:
        key = id(layer)
        if key not in self.groups:
            self.groups[key] = SwapGroup(type(layer).__name__)
        return self.groups[key]

    def add_tensor(self, st: SwapTensor) -> None:
        if self.current is not None:
            self.group_of(self.current).add(st)

    # Groups driven by hand under a name of the caller's choosing -- the reference's manual interface
    # (core/activation_checkpoint/swap.py:267-309 there): collect tensors with ``add_storage``, then
    # ``launch_offload`` / ``wait_offload`` after the forward and ``launch_load`` / ``wait_load`` before
    # the backward of the layer they belong to.
    def _named(self, group_name: str, create: bool = False) -> SwapGroup:
        named = self.__dict__.setdefault("named_groups", {})
        if group_name not in named:
            if not create:
                raise RuntimeError(f"Group {group_name} does not exist.")
            named[group_name] = SwapGroup(group_name)
        return named[group_name]

    def add_storage(self, group_name: str, storage) -> None:
        self._named(group_name, create=True).add(storage.swap_tensor if isinstance(storage, Storage) else storage)

    def launch_offload(self, group_name: str, copy_stream=None) -> None:
        self._named(group_name).launch_offload()

    def wait_offload(self, group_name: str) -> None:
        self._named(group_name).wait_offload()

    def launch_load(self, group_name: str, copy_stream=None) -> None:
        self._named(group_name).launch_load()

    def wait_load(self, group_name: str) -> None:
        self._named(group_name).wait_load()

    def get_current_group_name(self) -> str:
        return self.__dict__.get("current_group_name", "")

    def set_current_group_name(self, group_name: str) -> None:
        self.__dict__["current_group_name"] = group_name

    def set_forward_prefetch_layer(self, layer, next_layer) -> None:
        """Overlap ``layer``'s offload with ``next_layer``'s forward and its reload with
        ``next_layer``'s backward."""
        mgr = self
        mgr._prev_of[id(next_layer)] = layer

        def fwd_pre(mod, args):
            mgr.current = mod
            mgr.group_of(mod).clear()

        def fwd_post(mod, args, out):
            mgr.current = None
            mgr.group_of(mod).launch_offload()          # offload me while the next layer computes
            prev = mgr._prev_of.get(id(mod))
            if prev is not None:
                mgr.group_of(prev).wait_offload()       # the layer before me must be done by now
            return out

        def bwd_pre(mod, grad_out):
            prev = mgr._prev_of.get(id(mod))
            if prev is not None:
                mgr.group_of(prev).launch_load()        # fetch the previous layer while I run backward
            mgr.group_of(mod).wait_load()

        for m in (layer, next_layer):
            if not getattr(m, "_swap_hooks_installed", False):
                m.register_forward_pre_hook(fwd_pre)
                m.register_forward_hook(fwd_post)
                m.register_full_backward_pre_hook(bwd_pre)
                m._swap_hooks_installed = True

    def reset(self) -> None:
        self.groups.clear()
        self._prev_of.clear()
        self.current = None
        self.__dict__.pop("named_groups", None)
        self.__dict__.pop("current_group_name", None)
