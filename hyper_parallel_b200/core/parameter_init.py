"""``init_parameters``: deferred parameter initialisation after sharding.

Entry point of hyper_parallel/core/parameter_init.py:16-29 of the reference, whose
torch platform only validated its arguments.  Here it is implemented for torch:

1. build the model on the ``meta`` device (no memory), apply ``shard_module`` / ``hsdp``;
2. ``init_parameters(model)`` walks the modules in ``model.modules()`` order; for each
   module with parameters it materialises the module's **full** parameters one module at a
   time, runs the module's own ``reset_parameters()`` (or ``init_fn(module)``) on them with
   the process-wide RNG -- seeded identically on every rank -- and keeps only this rank's
   slice (TP layout slice, then HSDP dim-0 chunk).

Because every rank draws the same full tensors in the same order as a single-process
``reset_parameters`` walk, each shard equals the corresponding slice of the single-process
initialisation.  Peak extra memory is one module's full parameters.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
from torch import nn

from .dtensor import DTensor


def _global_shape(p: nn.Parameter):
    hp = getattr(p, "_hsdp_param", None)
    local_full = hp.full_shape if hp is not None else tuple((p._local_tensor if isinstance(p, DTensor) else p).shape)
    if isinstance(p, DTensor):
        return tuple(p.layout.get_global_shape(local_full))
    return tuple(local_full)


def _local_slice(p: nn.Parameter, full: torch.Tensor) -> torch.Tensor:
    t = full
    if isinstance(p, DTensor):
        area = p.layout.slice_area(full.shape)
        t = t[tuple(slice(b, e) for b, e in area)]
    hp = getattr(p, "_hsdp_param", None)
    if hp is not None and hp.sharded:
        t = t.chunk(hp.shard_size, dim=0)[hp.sharded_group_info.index]
    return t


def _materialise(root: nn.Module, p: nn.Parameter, value: torch.Tensor) -> None:
    """Store ``value`` (this rank's shard) as the data of ``p``; a meta parameter is replaced by a
    new parameter object on the target device (every alias in ``root`` is re-pointed)."""
    hp = getattr(p, "_hsdp_param", None)
    leaf = p._local_tensor if isinstance(p, DTensor) else p
    if leaf.device.type != "meta":
        with torch.no_grad():
            (hp.shard if hp is not None else leaf.data).copy_(value)
        return
    new_data = value.detach().clone()
    if isinstance(p, DTensor):
        new_p = nn.Parameter(DTensor._wrap(new_data, p.layout), requires_grad=leaf.requires_grad)
    else:
        new_p = nn.Parameter(new_data, requires_grad=p.requires_grad)
    for k, v in p.__dict__.items():
        if k not in ("_local_tensor", "_layout", "_hsdp_param"):
            try:
                setattr(new_p, k, v)
            except AttributeError:
                pass
    for m in root.modules():
        for n, q in list(m._parameters.items()):
            if q is p:
                m._parameters[n] = new_p
    if hp is not None:
        hp.rebind_param(new_p)


def init_parameters(module: nn.Module, stage_index: int = 0, *, device=None,
                    init_fn: Optional[Callable[[nn.Module], None]] = None,
                    seed: Optional[int] = None) -> nn.Module:
    """Materialise and initialise the (sharded) parameters of ``module`` in place; returns ``module``
    (the reference's README writes ``model = init_parameters(model)``).

    Args:
        stage_index: pipeline stage of this module; added to ``seed`` so that stages draw
            different streams when a seed is given.
        device: where the shards live afterwards (default: CUDA device if available, else CPU).
        init_fn: ``init_fn(submodule)`` initialises the submodule's own full parameters; default is
            ``submodule.reset_parameters()``.
        seed: re-seed the global RNG with ``seed + stage_index`` first.
    """
    if not isinstance(module, nn.Module):
        raise ValueError(f"init_parameters expects a torch.nn.Module, but got {type(module)}")
    if not isinstance(stage_index, int) or stage_index < 0:
        raise ValueError(f"stage_index must be a non-negative integer, but got {stage_index}")
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() \
            else torch.device("cpu")
    device = torch.device(device)
    if seed is not None:
        torch.manual_seed(seed + stage_index)
    done = set()
    for sub in module.modules():
        own = [(n, p) for n, p in sub._parameters.items() if p is not None and id(p) not in done]
        own_buffers = [(n, b) for n, b in sub._buffers.items() if b is not None and b.device.type == "meta"]
        if not own and not own_buffers:
            continue
        fn = init_fn if init_fn is not None else getattr(sub, "reset_parameters", None)
        if fn is None and own:
            raise RuntimeError(f"{type(sub).__name__} has parameters but no reset_parameters(); pass init_fn")
        saved = {}
        for n, p in own:
            done.add(id(p))
            saved[n] = p
            full = torch.empty(_global_shape(p), dtype=p.dtype, device=device)
            sub._parameters[n] = nn.Parameter(full, requires_grad=p.requires_grad)
        for n, b in own_buffers:
            sub._buffers[n] = torch.empty(b.shape, dtype=b.dtype, device=device)
        try:
            with torch.no_grad():
                if init_fn is not None:
                    init_fn(sub)
                elif fn is not None:
                    fn()
            fulls = {n: sub._parameters[n].detach() for n, _ in own}
        finally:
            for n, p in saved.items():
                sub._parameters[n] = p
        for n, p in own:
            _materialise(module, p, _local_slice(p, fulls[n]).to(device))
    for sub in module.modules():
        sch = sub.__dict__.get("hsdp_scheduler")
        if sch is not None:
            sch.hsdp_state.rebuild_param_buffers()
            sch._bind_symm_buffers()
    return module
