"""Gradient reduction of HSDP parameters (synchronous and asynchronous).

The case matrix is the one of hyper_parallel/core/hsdp/hsdp_grad_hook.py:19-166 and
hsdp_async_grad_hook.py:20-142 of the reference:

============================  =========================================================
parameter                     reduction
============================  =========================================================
unsharded, 1 replica          scale only
unsharded, n replicas         all-reduce over the replica group
fully sharded                 reduce-scatter over the shard group
partially sharded             reduce-scatter over the shard group, then all-reduce over
                              the replica group
============================  =========================================================

with gradient accumulation: level1 accumulates the *full* gradient and reduces on the
sync step; level2/3 reduce-scatter every micro-step, accumulate the shard and
all-reduce across replicas only on the sync step.  ``reduce_dtype`` casts before the
collective and back after it; ``grad_scale`` multiplies after the reduce.

Asynchronous mode launches the collectives with ``async_op=True``; the pending handle
and its post-processing are queued on the scheduler and drained by
``hsdp_sync_stream()`` (or when the next reduction of the same parameter arrives).
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch

from ...collectives import cc
from .hsdp_param import HSDPParam
from .hsdp_utils import HSDPConfig, OptimizerLevel


class PendingReduce:
    """An in-flight gradient reduction: wait for the handles, then run ``post``."""

    def __init__(self, works: List[object], post: Callable[[], None]):
        self.works = [w for w in works if w is not None]
        self.post = post

    def wait(self) -> None:
        for w in self.works:
            w.wait()
        self.post()


class HSDPGradHook:
    """Turns a freshly accumulated full gradient into the final (shard-shaped) gradient."""

    def __init__(self, config: HSDPConfig):
        self.config = config
        self.requires_grad_sync = True

    def set_requires_grad_sync(self, flag: bool) -> None:
        self.requires_grad_sync = bool(flag)

    # -- helpers ----------------------------------------------------------------
    def _cast_in(self, g: torch.Tensor) -> torch.Tensor:
        rd = self.config.reduce_dtype
        return g.to(rd) if rd is not None and g.dtype != rd else g

    def _finish(self, hp: HSDPParam, out: torch.Tensor, orig_dtype: torch.dtype) -> None:
        if out.dtype != orig_dtype:
            out = out.to(orig_dtype)
        if self.config.grad_scale != 1.0:
            out = out * self.config.grad_scale
        hp.reduced_grad = out

    def _reduce_scatter(self, hp: HSDPParam, g: torch.Tensor, works: list) -> torch.Tensor:
        out = torch.empty(hp.shard_shape, dtype=g.dtype, device=g.device)
        works.append(cc.reduce_scatter_into(out, g, hp.sharded_group_info.group, "sum",
                                            async_op=self.config.comm_async))
        return out

    def _all_reduce(self, hp: HSDPParam, g: torch.Tensor, works: list) -> torch.Tensor:
        if hp.dp_size > 1:
            if works and self.config.comm_async:
                # the all-reduce consumes the reduce-scatter output: order them on the handle
                for w in works:
                    if w is not None:
                        w.wait()
                works.clear()
            works.append(cc.all_reduce_(g, "sum", hp.unsharded_group_info.group,
                                        async_op=self.config.comm_async))
        return g

    # -- main entry ---------------------------------------------------------------
    def process(self, hp: HSDPParam, grad: torch.Tensor) -> Optional[PendingReduce]:
        """Reduce ``grad`` (full local shape).  Sets ``hp.reduced_grad`` now (sync) or when the
        returned :class:`PendingReduce` is waited (async).  ``reduced_grad`` stays ``None`` on
        a non-sync micro-step."""
        cfg = self.config
        orig_dtype = grad.dtype
        acc = cfg.requires_acc_grad
        sync = self.requires_grad_sync
        level1 = cfg.shard_level == OptimizerLevel.SHARD_OPT
        works: list = []
        hp.reduced_grad = None

        if not hp.sharded:
            g = grad
            if acc:
                g = hp.ensure_acc_grad(grad).add_(grad)
                if not sync:
                    return None
            if hp.dp_size == 1:
                self._finish(hp, g if not acc else g.clone(), orig_dtype)
                return None
            g = self._cast_in(g if not acc else g.clone())   # a fresh .grad tensor is ours to reduce in place
            out = self._all_reduce(hp, g, works)
        elif acc and level1:
            full = hp.ensure_acc_grad(grad).add_(grad)
            if not sync:
                return None
            out = self._reduce_scatter(hp, self._cast_in(full), works)
            out = self._all_reduce(hp, out, works)
        else:
            out = self._reduce_scatter(hp, self._cast_in(grad), works)
            if acc:
                # the accumulation needs the reduce-scatter result
                for w in works:
                    if w is not None:
                        w.wait()
                works.clear()
                shard_acc = hp.ensure_acc_grad(out).add_(out)
                if not sync:
                    return None
                out = self._all_reduce(hp, shard_acc.clone(), works)
            else:
                out = self._all_reduce(hp, out, works)

        if any(w is not None for w in works):
            return PendingReduce(works, lambda: self._finish(hp, out, orig_dtype))
        self._finish(hp, out, orig_dtype)
        return None


HSDPAsyncGradHook = HSDPGradHook  # asynchronous behaviour is selected by ``config.comm_async``
