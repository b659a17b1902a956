"""AdamW with fp32 master weights on (sharded) bf16 parameters, one fused kernel per tensor.

The reference has no optimizer of its own (its tests use ``torch.optim.SGD``); this one
exists because the headline configuration trains bf16 weights with fp32 master states.
State per parameter shard: fp32 master copy, ``exp_avg``, ``exp_avg_sq``.

``fuse_into_backward(model)`` makes HSDP hand each reduced gradient shard to the optimizer
the moment it is ready, so the update overlaps the rest of backward and the gradient is
freed immediately; ``step()`` then only finishes the parameters that were not handled and
advances the step counter.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Iterable

import torch

from ..core.dtensor import DTensor
from ..ops import functional as Fn


def _leaf(p: torch.Tensor) -> torch.Tensor:
    return p._local_tensor if isinstance(p, DTensor) else p


class FusedAdamW(torch.optim.Optimizer):
    def __init__(self, params: Iterable, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 1e-2, master_weights: bool = True):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)
        self.master_weights = master_weights
        self._step_count = 0
        self._done_in_backward = set()
        self._fused_params = set()
        self._flat_states: Dict[int, dict] = {}
        self._buffer_groups: Dict[int, list] = {}
        self._group_of: Dict[int, dict] = {}
        for g in self.param_groups:
            for p in g["params"]:
                self._group_of[id(p)] = g

    # -------------------------------------------------------------- state --
    def _state_for(self, p) -> dict:
        st = self.state[p]
        if not st:
            data = _leaf(p).data
            keep_master = self.master_weights and data.dtype != torch.float32
            st["master"] = data.detach().float().clone() if keep_master else None
            st["exp_avg"] = torch.zeros(data.shape, dtype=torch.float32, device=data.device)
            st["exp_avg_sq"] = torch.zeros(data.shape, dtype=torch.float32, device=data.device)
        return st

    def init_state(self) -> None:
        """Allocate all optimizer state now (instead of lazily on the first step)."""
        for g in self.param_groups:
            for p in g["params"]:
                if not p.requires_grad:
                    continue
                hp = getattr(p, "_hsdp_param", None)
                symm = getattr(hp, "_symm", None) if hp is not None else None
                if symm is not None and symm[0].optimizer is self:
                    self.flat_state_for(symm[0])
                else:
                    self._state_for(p)

    def _update(self, p, grad: torch.Tensor, step: int) -> None:
        g = self._group_of[id(p)]
        st = self._state_for(p)
        data = _leaf(p).data
        grad = grad.reshape(data.shape)
        if not grad.is_contiguous():
            grad = grad.contiguous()
        master = st["master"]
        if master is None:
            # fp32 parameters: the parameter itself is the master copy
            if data.is_cuda:
                Fn.adamw_step_(None, data.view(-1), st["exp_avg"].view(-1), st["exp_avg_sq"].view(-1),
                               grad.view(-1), lr=g["lr"], beta1=g["betas"][0], beta2=g["betas"][1],
                               eps=g["eps"], weight_decay=g["weight_decay"], step=step)
            else:
                Fn.adamw_step_(None, data.view(-1), st["exp_avg"].view(-1), st["exp_avg_sq"].view(-1),
                               grad.reshape(-1), lr=g["lr"], beta1=g["betas"][0], beta2=g["betas"][1],
                               eps=g["eps"], weight_decay=g["weight_decay"], step=step)
            return
        Fn.adamw_step_(data.view(-1), master.view(-1), st["exp_avg"].view(-1), st["exp_avg_sq"].view(-1),
                       grad.view(-1) if grad.is_contiguous() else grad.reshape(-1),
                       lr=g["lr"], beta1=g["betas"][0], beta2=g["betas"][1], eps=g["eps"],
                       weight_decay=g["weight_decay"], step=step)

    # ------------------------------------------------------- backward fusion --
    def fuse_into_backward(self, model: torch.nn.Module) -> None:
        """Consume each HSDP-reduced gradient as soon as it exists (update overlaps backward).

        Parameters held in symmetric-memory buffers are updated by the fused reduce-scatter +
        AdamW kernel (one launch per wrapped module); the others by one AdamW launch each."""
        for p in model.parameters():
            hp = getattr(p, "_hsdp_param", None)
            if hp is None or id(p) not in self._group_of:
                continue
            symm = getattr(hp, "_symm", None)
            if symm is not None and self._attach_buffer(symm[0]):
                self._fused_params.add(id(p))
            elif symm is None:
                hp.grad_consumer = self._consume

    def _attach_buffer(self, buf) -> bool:
        """Let the fused reduce-scatter + AdamW kernel update ``buf``.  Its parameters may belong to
        different parameter groups (no weight decay on the norm weights, per-group learning rates):
        every segment of the flat buffer carries the index of its group's row in the hyper-parameter
        table of the launch.  A buffer whose parameters are not all in this optimizer, or span more
        groups than the table holds, is left to the unfused path."""
        if buf.optimizer is self:
            return True
        groups, index = [], []
        for hp in buf.params:
            g = self._group_of.get(id(hp.param))
            if g is None:
                return False
            for k, have in enumerate(groups):
                if have is g:
                    index.append(k)
                    break
            else:
                groups.append(g)
                index.append(len(groups) - 1)
        if len(groups) > 4:
            return False
        buf.optimizer = self
        buf.set_param_groups(index)
        self._buffer_groups[id(buf)] = groups
        return True

    def flat_state_for(self, buf) -> dict:
        """fp32 master / moments for the flat shard of a symmetric buffer."""
        st = self._flat_states.get(id(buf))
        if st is None:
            st = {"master": buf.flat_shard.float().clone(),
                  "exp_avg": torch.zeros(buf.shard_numel, dtype=torch.float32, device=buf.device),
                  "exp_avg_sq": torch.zeros(buf.shard_numel, dtype=torch.float32, device=buf.device)}
            self._flat_states[id(buf)] = st
        return st

    def hyper_table_for(self, buf):
        """``{lr, beta1, beta2, eps, weight_decay}`` of every parameter group of ``buf`` (ctypes floats,
        read at launch time so that schedulers that change ``lr`` are honoured)."""
        groups = self._buffer_groups[id(buf)]
        vals = []
        for g in groups:
            vals += [g["lr"], g["betas"][0], g["betas"][1], g["eps"], g["weight_decay"]]
        return (ctypes.c_float * len(vals))(*vals)

    def _consume(self, hp, grad: torch.Tensor) -> None:
        p = hp.param
        self._update(p, grad, self._step_count + 1)
        self._done_in_backward.add(id(p))

    # ------------------------------------------------------------------ step --
    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        self._step_count += 1
        for g in self.param_groups:
            for p in g["params"]:
                if id(p) in self._done_in_backward or id(p) in self._fused_params:
                    continue
                grad = _leaf(p).grad
                if grad is None:
                    continue
                self._update(p, grad, self._step_count)
        self._done_in_backward.clear()
        return loss

    def zero_grad(self, set_to_none: bool = True) -> None:
        for g in self.param_groups:
            for p in g["params"]:
                lf = _leaf(p)
                if lf.grad is not None:
                    if set_to_none:
                        lf.grad = None
                    else:
                        lf.grad.zero_()
