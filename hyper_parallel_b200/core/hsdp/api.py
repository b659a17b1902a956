"""``hsdp()``: ZeRO-1/2/3 and hybrid sharded data parallel for any ``nn.Module``.

API of hyper_parallel/core/hsdp/api.py:162-272 of the reference.  The module's class is
replaced by a dynamic ``HSDP<Cls>(HSDPCell, Cls)`` so that the instance gains
``set_requires_grad_sync``, ``zero_grads``, ``set_forward_prefetch_cells`` and
``set_backward_prefetch_cells``.  Nested use is supported: wrap the blocks first, then the
root -- each call only manages the parameters that no earlier call has taken.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .hsdp_scheduler import HSDPScheduler, hsdp_sync_stream  # noqa: F401
from .hsdp_utils import HSDPConfig, OptimizerLevel


class HSDPCell:
    """Mix-in carrying the HSDP controls of a wrapped module."""

    hsdp_scheduler: HSDPScheduler

    def _hsdp_schedulers(self):
        seen = []
        for m in self.modules():
            sch = m.__dict__.get("hsdp_scheduler")
            if sch is not None:
                seen.append(sch)
        return seen

    def set_requires_grad_sync(self, requires_grad_sync: bool) -> None:
        """``False`` = accumulate locally on this micro-step, ``True`` = reduce (the sync step)."""
        for sch in self._hsdp_schedulers():
            sch.set_requires_grad_sync(requires_grad_sync)

    def zero_grads(self) -> None:
        """Clear accumulated and installed gradients."""
        for sch in self._hsdp_schedulers():
            sch.zero_grads()

    def set_forward_prefetch_cells(self, hsdp_cell_list) -> None:
        """Cells whose parameters are gathered asynchronously while this cell runs forward."""
        _check_cells(hsdp_cell_list)
        self.hsdp_scheduler.set_forward_prefetch_cells(hsdp_cell_list)

    def set_backward_prefetch_cells(self, hsdp_cell_list) -> None:
        """Cells whose parameters are gathered asynchronously while this cell runs backward."""
        _check_cells(hsdp_cell_list)
        self.hsdp_scheduler.set_backward_prefetch_cells(hsdp_cell_list)


def _check_cells(cells) -> None:
    if not isinstance(cells, (list, tuple)):
        raise ValueError("prefetch cells must be given as a list or tuple of HSDP cells")
    for c in cells:
        if not isinstance(c, HSDPCell):
            raise ValueError(f"prefetch cell {type(c).__name__} was not wrapped by hsdp()")


def _validate(cell, shard_size, threshold, optimizer_level, enable_grad_accumulation, grad_scale,
              reduce_dtype, comm_async, comm_fusion, bucket_size):
    if not isinstance(cell, nn.Module):
        raise ValueError(f"cell must be a torch.nn.Module, but got {type(cell)}")
    if not isinstance(shard_size, int) or isinstance(shard_size, bool) or (shard_size <= 0 and shard_size != -1):
        raise ValueError(f"shard_size must be a positive integer or -1, but got {shard_size}")
    if not isinstance(threshold, int) or isinstance(threshold, bool) or threshold < 0:
        raise ValueError(f"threshold must be a non-negative integer (KB), but got {threshold}")
    if optimizer_level not in ("level1", "level2", "level3"):
        raise ValueError(f"optimizer_level must be 'level1', 'level2' or 'level3', but got {optimizer_level!r}")
    for name, v in (("enable_grad_accumulation", enable_grad_accumulation), ("comm_async", comm_async),
                    ("comm_fusion", comm_fusion)):
        if not isinstance(v, bool):
            raise ValueError(f"{name} must be a bool, but got {type(v)}")
    if not isinstance(grad_scale, (int, float)) or isinstance(grad_scale, bool):
        raise ValueError(f"grad_scale must be a number, but got {type(grad_scale)}")
    if reduce_dtype is not None and not isinstance(reduce_dtype, torch.dtype):
        raise ValueError(f"reduce_dtype must be a torch.dtype or None, but got {reduce_dtype!r}")
    if not isinstance(bucket_size, int) or isinstance(bucket_size, bool) or bucket_size < -1:
        raise ValueError(f"bucket_size must be an integer >= -1 (KB), but got {bucket_size}")


def hsdp(cell: nn.Module, shard_size: int = -1, threshold: int = 64, optimizer_level: str = "level1",
         enable_grad_accumulation: bool = False, use_eager_hook: bool = True, grad_scale: float = 1.0,
         reduce_dtype: Optional[torch.dtype] = None, comm_async: bool = False,
         comm_fusion: bool = False, bucket_size: int = -1) -> nn.Module:
    """Shard ``cell``'s parameters, gradients and (implicitly) optimizer state over data-parallel ranks.

    Args:
        shard_size: ranks per shard group (``-1`` = as many as divide the parameter); the remaining
            data-parallel ranks replicate (HSDP).  ``1`` = pure data parallel.
        threshold: parameters smaller than this many KB are not sharded.
        optimizer_level: ``"level1"`` shard optimizer state and weights, ``"level2"`` also gradients,
            ``"level3"`` also re-gather the weights in backward.
        enable_grad_accumulation: keep accumulation buffers; use ``set_requires_grad_sync``.
        grad_scale: multiplied into the reduced gradient.
        reduce_dtype: dtype of the gradient collectives.
        comm_async: asynchronous gradient reduction; call ``hsdp_sync_stream()`` before the optimizer.
        comm_fusion / bucket_size: fuse parameter gathers into flat buffers and gradient reductions
            into buckets of ``bucket_size`` KB (``-1`` = one bucket per group, ``0`` = no gradient fusion).
    """
    _validate(cell, shard_size, threshold, optimizer_level, enable_grad_accumulation, grad_scale,
              reduce_dtype, comm_async, comm_fusion, bucket_size)
    config = HSDPConfig(
        shard_size=shard_size, threshold=threshold * 1024, shard_level=OptimizerLevel(optimizer_level),
        requires_acc_grad=enable_grad_accumulation, grad_scale=float(grad_scale), reduce_dtype=reduce_dtype,
        comm_async=comm_async, comm_fusion=comm_fusion,
        bucket_size=bucket_size * 1024 if bucket_size > 0 else bucket_size, use_eager_hook=use_eager_hook)
    params = []
    seen = set()
    for name, p in cell.named_parameters():
        if id(p) in seen or getattr(p, "_hsdp_param", None) is not None:
            continue
        if getattr(p, "hsdp_ignore", False):
            # not data-parallel state at all (e.g. expert-parallel weights: every rank owns different
            # experts): left alone -- no sharding, no gradient synchronisation
            continue
        seen.add(id(p))
        params.append((name, p))
    cls = cell.__class__
    if not isinstance(cell, HSDPCell):
        cell.__class__ = type(f"HSDP{cls.__name__}", (HSDPCell, cls), {})
    cell.__dict__["hsdp_scheduler"] = HSDPScheduler(cell, config, params)
    return cell
