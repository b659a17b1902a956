"""Sharded state dicts of ``hsdp()``-wrapped models and their optimizer, for distributed checkpoints.

``hsdp`` shards plain parameters along dim 0 over the shard group; nothing in the parameter itself
says so, hence a state dict of raw shards could not be loaded on another number of ranks.
``get_sharded_state_dict`` describes every shard as a DTensor over a 1-D mesh of its shard group
(aliasing the live storage), adds the optimizer state (fp32 master / exp_avg / exp_avg_sq of
:class:`~hyper_parallel_b200.optim.FusedAdamW`, which are sharded like the parameter) and the step
count.  ``core.checkpoint.save`` then writes it with global shapes, and ``load`` fills the very
tensors the model and the optimizer use -- on any number of ranks.  The reference has no
optimizer-state helper (its checkpoint tests save parameters only).
"""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch

from ..dtensor import DTensor
from ..layout import Layout


def _as_dtensor(local: torch.Tensor, hp) -> Any:
    """DTensor view of a dim-0 HSDP shard; replicated parameters stay plain tensors."""
    if not hp.sharded:
        return local
    ranks = list(hp.sharded_group_info.ranks)
    lay = Layout((len(ranks),), ("hsdp",), ranks)
    spec = ("hsdp",) + ("None",) * (local.dim() - 1)
    return DTensor._wrap(local, lay(*spec))


def get_sharded_state_dict(model: torch.nn.Module, optimizer=None, prefix: str = "model.") -> Dict[str, Any]:
    """``{"model.<fqn>": shard, "optim.<fqn>.<state>": shard, "optim.step": int}`` aliasing live tensors."""
    out: Dict[str, Any] = {}
    for name, p in model.named_parameters():
        hp = getattr(p, "_hsdp_param", None)
        if isinstance(p, DTensor):
            if hp is not None and hp.sharded:
                raise NotImplementedError(f"{name}: DTensor parameters that hsdp shards further are not supported")
            out[prefix + name] = p
        elif hp is None:
            out[prefix + name] = p.data
        else:
            out[prefix + name] = _as_dtensor(hp.shard, hp)
        if optimizer is None:
            continue
        states = _optimizer_states(optimizer, p, hp)
        for key, t in states.items():
            if t is None:
                continue
            if isinstance(p, DTensor):
                out[f"optim.{name}.{key}"] = DTensor._wrap(t, p.layout)
            elif hp is None:
                out[f"optim.{name}.{key}"] = t
            else:
                out[f"optim.{name}.{key}"] = _as_dtensor(t, hp)
    for name, b in model.named_buffers():
        out[prefix + name] = b
    if optimizer is not None:
        out["optim.step"] = int(optimizer._step_count)
    return out


def _optimizer_states(optimizer, p, hp) -> Dict[str, Optional[torch.Tensor]]:
    symm = getattr(hp, "_symm", None) if hp is not None else None
    if symm is not None and getattr(symm[0], "optimizer", None) is optimizer:
        buf, i = symm
        st = optimizer.flat_state_for(buf)
        lo = buf.shard_off[i]
        hi = lo + hp.shard.numel()
        return {k: st[k][lo:hi].view(hp.shard.shape) for k in ("master", "exp_avg", "exp_avg_sq")}
    st = optimizer._state_for(p)
    return {k: st.get(k) for k in ("master", "exp_avg", "exp_avg_sq")}


def restore_optimizer_step(optimizer, state: Dict[str, Any]) -> None:
    """After ``checkpoint.load`` filled ``state`` in place: restore the scalar step count."""
    if "optim.step" in state:
        optimizer._step_count = int(state["optim.step"])
