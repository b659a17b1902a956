"""``custom_shard``: run a function on local shards (``local_map``-style escape hatch).

As hyper_parallel/core/shard/local_func.py:26-128 of the reference: DTensor
arguments are (optionally) redistributed to ``in_placements``, the function runs on
their local tensors, and tensor outputs are re-wrapped with ``out_placements``.
"""
from __future__ import annotations

from functools import wraps
from typing import Callable, Optional, Sequence

import torch

from ..device_mesh import DeviceMesh
from ..dtensor import DTensor, _build_layout
from ..layout import Layout


def _as_layout(spec, mesh, ndim):
    if spec is None:
        return None
    if isinstance(spec, Layout):
        lay = spec
        if lay._dim_axes is None:
            lay = lay.copy()
            lay.placement_to_tensor_map(ndim)
        return lay
    return _build_layout(mesh, tuple(spec), ndim)


def custom_shard(func: Callable, device_mesh: DeviceMesh, out_placements,
                 in_placements: Optional[Sequence] = None, redistribute_inputs: bool = True) -> Callable:
    """Wrap ``func`` so it computes on local tensors.

    Args:
        out_placements: placements (or Layout) of the single output, or a tuple with one entry per
            output (``None`` for non-tensor outputs).
        in_placements: one entry per positional argument (``None`` = leave as is).
        redistribute_inputs: redistribute a DTensor whose placements differ from ``in_placements``;
            when ``False`` a mismatch raises.
    """
    def single(spec) -> bool:
        from ..placement_types import Placement
        return isinstance(spec, Layout) or (isinstance(spec, (tuple, list)) and len(spec) > 0
                                            and isinstance(spec[0], Placement))

    @wraps(func)
    def wrapper(*args, **kwargs):
        local_args = []
        for i, a in enumerate(args):
            if isinstance(a, DTensor):
                spec = in_placements[i] if in_placements is not None and i < len(in_placements) else None
                if spec is not None:
                    want = _as_layout(spec, device_mesh, a.dim())
                    if a.layout != want:
                        if not redistribute_inputs:
                            raise ValueError(f"argument {i} has placements {a.placements}, expected "
                                             f"{want.placements}; set redistribute_inputs=True")
                        a = a.redistribute(want)
                local_args.append(a.to_local())
            else:
                local_args.append(a)
        local_kwargs = {k: (v.to_local() if isinstance(v, DTensor) else v) for k, v in kwargs.items()}
        out = func(*local_args, **local_kwargs)
        if out_placements is None:
            return out
        if isinstance(out, (tuple, list)):
            specs = [out_placements] * len(out) if single(out_placements) else list(out_placements)
            if len(specs) != len(out):
                raise ValueError(f"func returned {len(out)} outputs but out_placements has {len(specs)}")
            return type(out)(
                DTensor._wrap(o, _as_layout(s, device_mesh, o.dim()))
                if (s is not None and isinstance(o, torch.Tensor)) else o
                for o, s in zip(out, specs))
        if not isinstance(out, torch.Tensor):
            return out
        spec = out_placements if single(out_placements) else out_placements[0]
        return DTensor._wrap(out, _as_layout(spec, device_mesh, out.dim()))
    return wrapper
