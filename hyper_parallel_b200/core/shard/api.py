"""``shard_module`` / ``shard``: apply a :class:`ShardingPlan` to a module or callable.

Behaviour follows hyper_parallel/core/shard/api.py:368-467 of the reference: each
planned parameter is replaced by ``nn.Parameter(DTensor(local slice))``; forward
pre/post hooks redistribute DTensor inputs / outputs to the declared layouts;
modules listed in ``return_local_tensor`` hand back plain local tensors.  Unlike
the reference the (possibly unchanged) model is returned for world size 1 too.

The README spelling ``shard(model, {"forward": {"input": ..., "output": ...},
"parameter": {...}})`` is accepted by :func:`shard`.
"""
from __future__ import annotations

import inspect
from functools import wraps
from typing import Any, Callable, Dict, Optional, Union

import torch
from torch import nn

from ..device_mesh import DeviceMesh
from ..dtensor import DTensor, distribute_tensor
from ..layout import Layout
from ..placement_types import Placement
from .sharding_plan import ShardingPlan


# ----------------------------------------------------------- spec -> Layout --
def _is_spec(value) -> bool:
    """True for ONE layout spec: tuple of placements, or of aliases / tuples of aliases."""
    if isinstance(value, Layout):
        return True
    if not isinstance(value, tuple) or len(value) == 0:
        return False
    for item in value:
        if isinstance(item, (Placement, str)):
            continue
        if isinstance(item, tuple) and len(item) > 0 and all(isinstance(x, str) for x in item):
            continue
        return False
    return True


def _to_layout(spec, mesh: DeviceMesh) -> Layout:
    if isinstance(spec, Layout):
        return spec
    return Layout.from_device_mesh(mesh)(*spec) if not isinstance(spec[0], Placement) \
        else Layout.from_device_mesh(mesh)(spec)


def _convert_io(value, mesh):
    """-> None | list[Layout|None] | dict[str, Layout|None]"""
    if value is None:
        return None
    if isinstance(value, dict):
        return {k: (None if v is None else _to_layout(v, mesh)) for k, v in value.items()}
    if _is_spec(value):
        return [_to_layout(value, mesh)]
    if isinstance(value, (list, tuple)):
        return [None if v is None else _to_layout(v, mesh) for v in value]
    raise TypeError(f"unsupported layout specification {value!r}")


def _redistribute(t, layout: Optional[Layout]):
    if layout is None or not isinstance(t, DTensor):
        return t
    return t.redistribute(layout)


def _parallel_in(func, args, kwargs, layouts):
    args, kwargs = list(args), dict(kwargs)
    if isinstance(layouts, dict):
        names = list(inspect.signature(func).parameters.keys())
        for i, a in enumerate(args):
            if i < len(names) and names[i] in layouts:
                args[i] = _redistribute(a, layouts[names[i]])
        for k in kwargs:
            if k in layouts:
                kwargs[k] = _redistribute(kwargs[k], layouts[k])
    else:
        for i, a in enumerate(args):
            if i < len(layouts):
                args[i] = _redistribute(a, layouts[i])
    return tuple(args), kwargs


def _parallel_out(outputs, layouts):
    if isinstance(outputs, (tuple, list)):
        if len(outputs) != len(layouts):
            raise ValueError(f"The size of outputs and out_layout must be equal, but got {len(outputs)} "
                             f"and {len(layouts)}")
        return type(outputs)(_redistribute(o, l) for o, l in zip(outputs, layouts))
    if len(layouts) != 1:
        raise ValueError(f"The size of outputs and out_layout must be equal, but got 1 and {len(layouts)}")
    return _redistribute(outputs, layouts[0])


def _to_local_tree(out):
    if isinstance(out, DTensor):
        return out.to_local()
    if isinstance(out, (tuple, list)):
        return type(out)(_to_local_tree(o) for o in out)
    if isinstance(out, dict):
        return {k: _to_local_tree(v) for k, v in out.items()}
    return out


# ------------------------------------------------------------------- module --
def _set_parameter(model: nn.Module, fqn: str, new_param: nn.Parameter) -> None:
    parts = fqn.split(".")
    mod = model
    for p in parts[:-1]:
        mod = getattr(mod, p)
    old = mod._parameters.get(parts[-1])
    if old is None:
        raise ValueError(f"{fqn} is configured with a layout, but no instance was found.")
    # tied weights: replace every alias of the old parameter
    for m in model.modules():
        for n, p in list(m._parameters.items()):
            if p is old:
                m._parameters[n] = new_param


def shard_parameter(param: torch.Tensor, layout: Layout) -> nn.Parameter:
    """Slice a full (replicated) parameter into this rank's shard wrapped as a DTensor parameter."""
    if isinstance(param, DTensor):
        return nn.Parameter(param.redistribute(layout).detach(), requires_grad=param.requires_grad)
    layout = layout.copy()
    layout.placement_to_tensor_map(param.dim())
    if param.device.type == "meta":
        local = torch.empty(layout.get_local_shape(param.shape), dtype=param.dtype, device="meta")
        dt = DTensor._wrap(local, layout)
    else:
        dt = distribute_tensor(param.detach(), layout)
    return nn.Parameter(dt, requires_grad=param.requires_grad)


def _register_hooks(model: nn.Module, forward_plan: Dict[str, Any], mesh: DeviceMesh) -> None:
    modules = dict(model.named_modules())
    for key, value in forward_plan.items():
        if value is None:
            continue
        prefix, _, suffix = key.rpartition(".")
        if suffix not in ("input", "output"):
            raise ValueError("In python shard_module, sharding_plan's forward key must end with input or "
                             f"output, but got type {suffix}")
        if prefix not in modules:
            raise ValueError(f"sharding plan names submodule {prefix!r} which does not exist")
        target = modules[prefix]
        layouts = _convert_io(value, mesh)
        if suffix == "input":
            target.in_layout = layouts

            def pre_hook(mod, args, kwargs):
                return _parallel_in(mod.forward, args, kwargs, mod.in_layout)
            target.register_forward_pre_hook(pre_hook, with_kwargs=True)
        else:
            if isinstance(layouts, dict):
                raise TypeError("output layouts must be a spec or a list of specs")
            target.out_layout = layouts

            def post_hook(mod, args, outputs):
                return _parallel_out(outputs, mod.out_layout)
            target.register_forward_hook(post_hook)


def shard_module(model: Union[nn.Module, Callable], device_mesh: DeviceMesh,
                 sharding_plan: ShardingPlan):
    """Shard ``model`` (module or plain callable) over ``device_mesh`` according to ``sharding_plan``."""
    if not isinstance(sharding_plan, ShardingPlan):
        raise TypeError("The 'sharding_plan' must be an instance of ShardingPlan, but got "
                        f"{type(sharding_plan)}. Direct dict input is not supported.")
    for name in ("input_plan", "output_plan"):
        v = getattr(sharding_plan, name)
        if v is not None and not isinstance(v, dict):
            raise TypeError(f"{name} must be a dict, but got {type(v)}")
    forward_plan: Dict[str, Any] = {}
    forward_plan.update(sharding_plan.input_plan or {})
    forward_plan.update(sharding_plan.output_plan or {})

    if not isinstance(model, nn.Module):
        in_l = _convert_io(forward_plan.get("input"), device_mesh)
        out_l = _convert_io(forward_plan.get("output"), device_mesh)
        if in_l is None and out_l is None:
            return model
        func = model

        @wraps(func)
        def wrapper(*args, **kwargs):
            if in_l is not None:
                args, kwargs = _parallel_in(func, args, kwargs, in_l)
            out = func(*args, **kwargs)
            if out_l is not None:
                out = _parallel_out(out, out_l)
            return out
        return wrapper

    for fqn, spec in (sharding_plan.plan or {}).items():
        layout = _to_layout(spec, device_mesh)
        params = dict(model.named_parameters(remove_duplicate=False))
        if fqn not in params:
            raise ValueError(f"{fqn} is configured with a layout, but no instance was found.")
        _set_parameter(model, fqn, shard_parameter(params[fqn], layout))
    if forward_plan:
        _register_hooks(model, forward_plan, device_mesh)
    if sharding_plan.return_local_tensor:
        modules = dict(model.named_modules())
        for name in sharding_plan.return_local_tensor:
            if name not in modules:
                raise ValueError(f"return_local_tensor names submodule {name!r} which does not exist")
            modules[name].register_forward_hook(lambda mod, args, out: _to_local_tree(out))
    return model


def shard(model, sharding_plan, device_mesh: Optional[DeviceMesh] = None):
    """README-style entry point.

    ``sharding_plan`` is a :class:`ShardingPlan` or a dict
    ``{"parameter": {...}, "forward": {"input": ..., "output": ..., "<sub>.input": ...}}`` whose
    specs may be ``Layout`` objects (then ``device_mesh`` is taken from them).
    """
    if isinstance(sharding_plan, dict):
        fwd = sharding_plan.get("forward") or {}
        plan = ShardingPlan(
            plan=sharding_plan.get("parameter"),
            input_plan={k: v for k, v in fwd.items() if k.endswith("input")} or None,
            output_plan={k: v for k, v in fwd.items() if k.endswith("output")} or None,
            return_local_tensor=sharding_plan.get("return_local_tensor"))
    else:
        plan = sharding_plan
    if device_mesh is None:
        def find(v):
            if isinstance(v, Layout):
                return v.mesh
            if isinstance(v, dict):
                v = list(v.values())
            if isinstance(v, (list, tuple)):
                for x in v:
                    m = find(x)
                    if m is not None:
                        return m
            return None
        device_mesh = find([plan.plan, plan.input_plan, plan.output_plan])
        if device_mesh is None:
            raise ValueError("shard() needs a device_mesh when the plan has no Layout objects")
    return shard_module(model, device_mesh, plan)


def parallelize_value_and_grad(fn: Callable, weights=None, sens=None, *, params=None,
                               loss_layout: Optional[Layout] = None):
    """Return ``f(*args) -> (outputs, grads)`` that seeds the backward with ``1 / repeat_num``.

    A loss replicated on ``repeat_num`` ranks would be counted that many times by the
    gradient reductions; seeding with ``1 / repeat_num`` makes the summed gradients equal
    the single-process ones (hyper_parallel/core/shard/api.py:470-577 of the reference, there
    a MindSpore ``GradOperation`` wrapper with the same arguments).

    ``weights`` (``params`` is the older spelling): the parameters to differentiate; without them
    the gradients are accumulated into ``.grad`` and ``grads`` is ``None``.  ``sens``: when ``fn``
    returns several outputs, one sensitivity per output (multiplied into the seed); without it only
    the first output is differentiated."""
    weights = params if weights is None else weights
    if isinstance(weights, torch.Tensor):
        weights = [weights]

    def wrapped(*args, **kwargs):
        out = fn(*args, **kwargs)
        outs = list(out) if isinstance(out, (tuple, list)) else [out]
        if sens is not None and len(sens) != len(outs):
            raise ValueError(f"sens has {len(sens)} entries but fn returned {len(outs)} outputs")
        locals_, seeds = [], []
        for i, o in enumerate(outs):
            if not isinstance(o, torch.Tensor):
                continue
            weight = (1.0 if i == 0 else 0.0) if sens is None else float(sens[i])
            if weight == 0.0:
                continue
            lay = o.layout if isinstance(o, DTensor) else loss_layout
            rep = lay.repeat_num() if lay is not None else 1
            local = o.to_local() if isinstance(o, DTensor) else o
            if local.requires_grad:
                locals_.append(local)
                seeds.append(torch.full_like(local, weight / rep))
        if weights is None:
            if locals_:
                torch.autograd.backward(locals_, grad_tensors=seeds)
            return out, None
        targets = [p.to_local() if isinstance(p, DTensor) else p for p in weights]
        grads = torch.autograd.grad(locals_, targets, grad_outputs=seeds, allow_unused=True)
        return out, grads
    return wrapped
