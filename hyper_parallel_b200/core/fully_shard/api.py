"""``fully_shard``: FSDP2-style per-module sharding (hyper_parallel/core/fully_shard/api.py:357-492).

A 1-D mesh shards over all its ranks (FSDP); a 2-D mesh replicates over dim 0 and shards over
dim 1 (HSDP).  The wrapped module gains the ``HSDPModule`` methods.  ``get_model_state_dict``
returns sharded (DTensor) or full state dicts, optionally on CPU.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch
from torch import nn

from ...collectives import cc
from ..device_mesh import DeviceMesh, init_device_mesh
from ..dtensor import DTensor
from .param import FSDPParam
from .state import FSDPState
from .utils import (CPUOffloadPolicy, FSDPMeshInfo, HSDPMeshInfo, MixedPrecisionPolicy, OffloadPolicy,
                    StateDictOptions)


class _UnshardHandle:
    def __init__(self, state: Optional[FSDPState]):
        self.state = state

    def wait(self) -> None:
        if self.state is not None:
            self.state.wait_for_unshard()
            self.state = None

    _hsdp_state = property(lambda self: self.state)       # the reference's attribute name


def _need_bool(name: str, value) -> bool:
    if not isinstance(value, bool):
        raise ValueError(f"{name} must be a bool, got {type(value).__name__}")
    return value


def _need_modules(name: str, modules) -> list:
    if not isinstance(modules, (list, tuple)):
        raise ValueError(f"{name} must be a list of fully_shard modules, got {type(modules).__name__}")
    for m in modules:
        if not isinstance(m, nn.Module) or "_fsdp_state" not in m.__dict__:
            raise ValueError(f"{name}: {type(m).__name__} is not a fully_shard module")
    return list(modules)


class _SchedulerView:
    """Read-only view of a module's :class:`FSDPState` under the attribute names of the reference's
    scheduler object (``module.hsdp_scheduler`` there: core/fully_shard/hsdp_scheduler.py:32-194 and
    hsdp_state.py:22-177), for code that inspects it: ``requires_grad_sync``, ``reshard_after_forward``,
    ``forward_prefetch_cells`` / ``backward_prefetch_cells``, ``config.reshard_after_forward``,
    ``scheduler_ctx.is_last_backward``, ``hsdp_state.{reduce_grads, requires_all_reduce,
    reshard_after_backward, is_shard}``."""

    def __init__(self, state: FSDPState):
        self._s = state

    requires_grad_sync = property(lambda self: self._s.requires_gradient_sync)
    reduce_grads = property(lambda self: self._s.requires_gradient_sync)
    requires_all_reduce = property(lambda self: self._s.requires_all_reduce)
    reshard_after_forward = property(lambda self: self._s.reshard_after_forward)
    reshard_after_backward = property(lambda self: self._s.reshard_after_backward)
    is_last_backward = property(lambda self: self._s.is_last_backward)
    is_shard = property(lambda self: self._s.is_sharded)
    forward_prefetch_cells = property(lambda self: list(self._s.fwd_prefetch))
    backward_prefetch_cells = property(lambda self: list(self._s.bwd_prefetch))
    hsdp_state = property(lambda self: self)
    config = property(lambda self: self)
    scheduler_ctx = property(lambda self: self)


class HSDPModule:
    """Methods added to a module by :func:`fully_shard`."""

    _fsdp_state: FSDPState

    @property
    def hsdp_scheduler(self) -> _SchedulerView:
        return _SchedulerView(self._fsdp_state)

    def _states(self, recurse: bool = True) -> List[FSDPState]:
        mods = self.modules() if recurse else [self]
        return [m._fsdp_state for m in mods if "_fsdp_state" in m.__dict__]

    def unshard(self, async_op: bool = False) -> Optional[_UnshardHandle]:
        self._fsdp_state.unshard(async_op=True)
        if async_op:
            return _UnshardHandle(self._fsdp_state)
        self._fsdp_state.wait_for_unshard()
        return None

    def reshard(self) -> None:
        self._fsdp_state.reshard()

    def set_requires_gradient_sync(self, requires_gradient_sync: bool, *, recurse: bool = True) -> None:
        for st in self._states(recurse):
            st.requires_gradient_sync = _need_bool("requires_gradient_sync", requires_gradient_sync)

    def set_requires_all_reduce(self, requires_all_reduce: bool, *, recurse: bool = True) -> None:
        for st in self._states(recurse):
            st.requires_all_reduce = _need_bool("requires_all_reduce", requires_all_reduce)

    def set_is_last_backward(self, is_last_backward: bool) -> None:
        for st in self._states():
            st.is_last_backward = _need_bool("is_last_backward", is_last_backward)

    def set_reshard_after_forward(self, reshard_after_forward: bool, recurse: bool = True) -> None:
        for st in self._states(recurse):
            st.reshard_after_forward = _need_bool("reshard_after_forward", reshard_after_forward)

    def set_reshard_after_backward(self, reshard_after_backward: bool, *, recurse: bool = True) -> None:
        for st in self._states(recurse):
            st.reshard_after_backward = _need_bool("reshard_after_backward", reshard_after_backward)

    def set_modules_to_forward_prefetch(self, modules: List[nn.Module]) -> None:
        self._fsdp_state.fwd_prefetch = _need_modules("modules_to_forward_prefetch", modules)

    def set_modules_to_backward_prefetch(self, modules: List[nn.Module]) -> None:
        self._fsdp_state.bwd_prefetch = _need_modules("modules_to_backward_prefetch", modules)

    def zero_grads(self) -> None:
        """Drop the accumulated (sharded) gradients of every wrapped module below this one.  The
        reference refuses this call on torch and points at ``optimizer.zero_grad()``
        (hyper_parallel/core/fully_shard/api.py:91-99); here it does the same job."""
        for p in self.parameters():
            p.grad = None
            fp = getattr(p, "_fsdp_param", None)
            if fp is not None and getattr(fp, "sharded_param", None) is not None:
                fp.sharded_param.grad = None

    def set_reduce_op_type(self, reduce_op_type: str) -> None:
        if reduce_op_type not in ("avg", "sum"):
            raise ValueError(f"reduce_op_type must be 'avg' or 'sum', got {reduce_op_type!r}")
        for st in self._states():
            st.reduce_op = reduce_op_type

    def load_state_dict(self, state_dict: Dict[str, Any], strict: bool = True, assign: bool = False):
        """Accepts DTensors, local-shape tensors or global-shape tensors (sliced to this rank's shard)."""
        own = dict(self.named_parameters())
        own.update(dict(self.named_buffers()))
        missing = [k for k in own if k not in state_dict]
        unexpected = [k for k in state_dict if k not in own]
        if strict and (missing or unexpected):
            raise RuntimeError(f"Error(s) in loading state_dict: missing keys {missing}, unexpected keys {unexpected}")
        with torch.no_grad():
            for k, v in state_dict.items():
                if k not in own:
                    continue
                dst = own[k]
                fp = getattr(dst, "_fsdp_param", None)
                if fp is None:
                    src = v.to_local() if isinstance(v, DTensor) else v
                    dst.data.copy_(src)
                    continue
                local = fp.sharded_local
                if isinstance(v, DTensor):
                    src = v.to_local()
                elif tuple(v.shape) == tuple(local.shape) and fp.n > 1:
                    src = v
                elif tuple(v.shape) == fp.full_shape:
                    src = v.chunk(fp.n, dim=fp.shard_dim)[fp.mesh_info.shard_rank] if fp.n > 1 else v
                else:
                    raise RuntimeError(f"size mismatch for {k}: got {tuple(v.shape)}, expected local "
                                       f"{tuple(local.shape)} or global {fp.full_shape}")
                local.data.copy_(src.to(local.dtype))
        return torch.nn.modules.module._IncompatibleKeys(missing, unexpected)


def _default_mesh() -> DeviceMesh:
    return init_device_mesh("cuda", (cc.get_world_size(),), mesh_dim_names=("fsdp",))


def fully_shard(module: nn.Module, *, mesh: Optional[DeviceMesh] = None,
                reshard_after_forward: Optional[bool] = None, shard_placement_fn=None,
                mp_policy: MixedPrecisionPolicy = MixedPrecisionPolicy(),
                offload_policy: OffloadPolicy = OffloadPolicy(), ignored_params=None, device=None) -> nn.Module:
    """Shard ``module``'s parameters (those no nested ``fully_shard`` call already took)."""
    if not isinstance(module, nn.Module):
        raise ValueError(f"fully_shard expects an nn.Module, got {type(module)}")
    mesh = mesh or _default_mesh()
    if mesh.ndim == 1:
        mesh_info = FSDPMeshInfo(mesh, 0)
    elif mesh.ndim == 2:
        mesh_info = HSDPMeshInfo(mesh, shard_mesh_dim=1, replicate_mesh_dim=0)
    else:
        raise ValueError(f"fully_shard expects a 1-D or 2-D mesh, got {mesh.ndim}-D")
    ignored = {id(p) for p in (ignored_params or [])}
    owners: Dict[int, list] = {}
    order: List[nn.Parameter] = []
    for mod in module.modules():
        if mod is not module and "_fsdp_state" in mod.__dict__:
            continue
        for name, p in mod._parameters.items():
            if p is None or id(p) in ignored or getattr(p, "_fsdp_param", None) is not None:
                continue
            # skip parameters that live inside an already wrapped submodule
            if id(p) not in owners:
                owners[id(p)] = []
                order.append(p)
            owners[id(p)].append((mod, name))
    managed_elsewhere = set()
    for sub in module.modules():
        if sub is not module and "_fsdp_state" in sub.__dict__:
            for p in sub.parameters():
                managed_elsewhere.add(id(p))
    dev = torch.device(device) if device is not None else None
    params = []
    for p in order:
        if id(p) in managed_elsewhere:
            continue
        target = dev or p.device
        if isinstance(offload_policy, CPUOffloadPolicy) and dev is None:
            # the shard lives on the host; gathered parameters live on the compute device
            target = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else p.device
        params.append(FSDPParam(owners[id(p)], p, mesh_info, mp_policy, offload_policy, shard_placement_fn, target))
    cls = module.__class__
    if not isinstance(module, HSDPModule):
        module.__class__ = type(f"HSDP{cls.__name__}", (HSDPModule, cls), {})
    module.__dict__["_fsdp_state"] = FSDPState(module, params, mp_policy,
                                               True if reshard_after_forward is None else bool(reshard_after_forward))
    return module


def hsdp_sync_stream() -> None:
    """Wait for every gradient reduction of ``fully_shard`` modules that is still in flight (the root
    backward callback already does so at the end of ``backward``; reference core/fully_shard/api.py:495-499)."""
    from .state import _drain
    _drain(0)


def get_model_state_dict(model: nn.Module, *, options: Optional[StateDictOptions] = None) -> Dict[str, Any]:
    """State dict of a ``fully_shard`` model (hyper_parallel/core/fully_shard/api.py:443-490).

    ==================  =============  ==========================================
    ``full_state_dict``  ``cpu_offload``  result
    ==================  =============  ==========================================
    False               False          DTensors (this rank's shards, no copy)
    False               True           DTensors whose local shard is on the host
    True                False          full tensors on every rank
    True                True           full tensors on the host, rank 0 only
    ==================  =============  ==========================================

    ``ignore_frozen_params`` drops parameters with ``requires_grad=False``.  Every rank must call
    this function when ``full_state_dict`` is set: the gathers are collective.
    """
    options = options or StateDictOptions()
    full = bool(getattr(options, "full_state_dict", False))
    to_cpu = bool(getattr(options, "cpu_offload", False))
    if getattr(options, "broadcast_from_rank0", False) and not full:
        raise ValueError("full_state_dict must be True when broadcast_from_rank0 is True.")
    skip_frozen = bool(getattr(options, "ignore_frozen_params", False))
    keep = not (full and to_cpu) or cc.get_rank() == 0
    out: Dict[str, Any] = {}
    entries = [(n, p, True) for n, p in model.named_parameters()] + \
              [(n, b, False) for n, b in model.named_buffers()]
    persistent = set(model.state_dict().keys())
    for name, p, is_param in entries:
        if name not in persistent or (is_param and skip_frozen and not p.requires_grad):
            continue
        fp = getattr(p, "_fsdp_param", None)
        if fp is None:
            v = p.detach()
        elif full:
            v = fp.full_tensor().detach()
        else:
            v = fp.sharded_param.detach()
        if not keep:
            continue
        if to_cpu:
            v = v.cpu() if not isinstance(v, DTensor) else DTensor._wrap(v.to_local().cpu(), v.layout)
        out[name] = v
    return out
