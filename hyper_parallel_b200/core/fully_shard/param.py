"""One parameter managed by ``fully_shard``.

Capability of hyper_parallel/platform/torch/fully_shard/param.py:41-785 of the reference: the
sharded parameter is an ``nn.Parameter(DTensor)`` swapped into the owning module(s); unsharding
all-gathers (asynchronously) into a buffer and swaps a plain full parameter in; the gathered
storage is dropped on reshard; mixed precision casts the shard to ``param_dtype`` before the
gather and reduces gradients in ``reduce_dtype``; gradients are reduce-scattered (``avg`` or
``sum``) over the shard group and all-reduced over the replicate group; CPU offload keeps the
shard (and its gradient) in pinned host memory.  Only even sharding is supported.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
from torch import nn

from ...collectives import cc
from ..dtensor import DTensor
from ..placement_types import Replicate, Shard
from .utils import CPUOffloadPolicy, DataParallelMeshInfo, MixedPrecisionPolicy, OffloadPolicy


class FSDPParam:
    def __init__(self, owners: List[Tuple[nn.Module, str]], param: nn.Parameter, mesh_info: DataParallelMeshInfo,
                 mp_policy: MixedPrecisionPolicy, offload_policy: OffloadPolicy, shard_placement_fn=None,
                 device: Optional[torch.device] = None):
        self.owners = owners
        self.mesh_info = mesh_info
        self.mp_policy = mp_policy
        self.offload = isinstance(offload_policy, CPUOffloadPolicy)
        self.pin = self.offload and offload_policy.pin_memory and torch.cuda.is_available()
        self.device = device if device is not None else param.device
        self.orig_dtype = param.dtype
        self.param_dtype = mp_policy.param_dtype or param.dtype
        self.reduce_dtype = mp_policy.reduce_dtype
        self.requires_grad = param.requires_grad
        n = mesh_info.shard_size
        placement = shard_placement_fn(param) if shard_placement_fn is not None else None
        self.shard_dim = placement.dim if placement is not None else 0
        self.full_shape = tuple(param.shape)
        if n > 1:
            if param.dim() == 0 or self.full_shape[self.shard_dim] % n:
                raise NotImplementedError(
                    f"fully_shard supports even sharding only: dim {self.shard_dim} of shape {self.full_shape} "
                    f"is not divisible by {n}")
        self.n = n
        data = param.detach()
        if n > 1:
            data = data.chunk(n, dim=self.shard_dim)[mesh_info.shard_rank].contiguous().clone()
        if self.offload:
            data = data.cpu()
            if self.pin:
                data = data.pin_memory()
        elif data.device != self.device and data.device.type != "meta":
            data = data.to(self.device)
        mesh = mesh_info.mesh
        placements = [Replicate()] * mesh.ndim
        if mesh_info.shard_mesh_dim is not None:
            placements[mesh_info.shard_mesh_dim] = Shard(self.shard_dim)
        self.sharded_param = nn.Parameter(DTensor.from_local(data, mesh, placements), requires_grad=self.requires_grad)
        self.sharded_param._fsdp_param = self
        self.unsharded_param = nn.Parameter(torch.empty(0, dtype=self.param_dtype, device=self.device),
                                            requires_grad=self.requires_grad)
        self.unsharded_param._fsdp_param = self
        self._gather = None          # (work, buffer)
        self.is_sharded = True
        self._pending_reduce = None
        self._swap(self.sharded_param)

    # ----------------------------------------------------------------- swaps --
    def _swap(self, p: nn.Parameter) -> None:
        for mod, name in self.owners:
            mod._parameters[name] = p

    @property
    def sharded_state(self):
        from .hsdp_utils import ShardedState
        return ShardedState.SHARDED if self.is_sharded else ShardedState.UNSHARDED

    @property
    def sharded_local(self) -> torch.Tensor:
        return self.sharded_param._local_tensor

    # --------------------------------------------------------------- unshard --
    def unshard(self, async_op: bool = False) -> None:
        if not self.is_sharded or self._gather is not None:
            return
        shard = self.sharded_local.data
        if self.offload:
            shard = shard.to(self.device, non_blocking=True)
        if shard.dtype != self.param_dtype:
            shard = shard.to(self.param_dtype)
        if self.n == 1:
            self._gather = (None, shard.reshape((1,) + tuple(shard.shape)))
            return
        buf = torch.empty((self.n,) + tuple(shard.shape), dtype=self.param_dtype, device=self.device)
        work = cc.all_gather_into(buf.view(self.n * shard.shape[0], *shard.shape[1:]) if shard.dim() > 0 else buf,
                                  shard, self.mesh_info.shard_group, async_op=async_op)
        self._gather = (work, buf)

    def wait_for_unshard(self) -> None:
        if not self.is_sharded:
            return
        if self._gather is None:
            self.unshard(async_op=False)
        work, buf = self._gather
        self._gather = None
        if work is not None:
            work.wait()
        d = self.shard_dim
        full = buf.movedim(0, d).reshape(self.full_shape) if self.n > 1 else buf[0]
        self.unsharded_param.data = full
        self._swap(self.unsharded_param)
        self.is_sharded = False

    def reshard(self) -> None:
        if self.is_sharded:
            return
        self._swap(self.sharded_param)
        self.unsharded_param.data = torch.empty(0, dtype=self.param_dtype, device=self.device)
        self.is_sharded = True

    # ----------------------------------------------------------------- grads --
    def reduce_grad(self, reduce_op: str = "avg", requires_all_reduce: bool = True) -> None:
        """Launch the reduction of ``unsharded_param.grad`` (asynchronously on CUDA)."""
        g = self.unsharded_param.grad
        self.unsharded_param.grad = None
        if g is None:
            return
        rd = self.reduce_dtype or g.dtype
        if g.dtype != rd:
            g = g.to(rd)
        works = []
        if self.n > 1:
            d = self.shard_dim
            shp = list(self.full_shape)
            chunks = g.reshape(shp[:d] + [self.n, shp[d] // self.n] + shp[d + 1:]).movedim(d, 0).contiguous()
            out = torch.empty(chunks.shape[1:], dtype=rd, device=g.device)
            works.append(cc.reduce_scatter_into(out, chunks, self.mesh_info.shard_group, reduce_op, async_op=True))
        else:
            out = g
        self._pending_reduce = (works, out, reduce_op, requires_all_reduce)

    def finish_reduce(self) -> None:
        if self._pending_reduce is None:
            return
        works, out, reduce_op, requires_all_reduce = self._pending_reduce
        self._pending_reduce = None
        for w in works:
            if w is not None:
                w.wait()
        if requires_all_reduce and self.mesh_info.replicate_size > 1:
            cc.all_reduce_(out, reduce_op, self.mesh_info.replicate_group)
        self.apply_reduced_grad(out)

    def apply_reduced_grad(self, g: torch.Tensor) -> None:
        leaf = self.sharded_local
        if self.mp_policy.apply_grad_on_fp32_main_grad:
            g32 = g.float()
            if self.offload:
                g32 = g32.to("cpu", non_blocking=False)
            mg = getattr(self.sharded_param, "main_grad", None)
            if mg is None:
                self.sharded_param.main_grad = g32.clone()
            else:
                mg.add_(g32)
            return
        if g.dtype != self.orig_dtype:
            g = g.to(self.orig_dtype)
        if self.offload:
            g = g.to("cpu")
        # ``param.grad`` of a sharded parameter is a DTensor with the parameter's layout, as in the
        # reference (platform/torch/fully_shard/param.py:120-172 there): the local tensor carries it
        g = g.reshape(leaf.shape)
        if leaf.grad is None:
            leaf.grad = DTensor._wrap(g, self.sharded_param._layout)
        else:
            acc = leaf.grad
            (acc._local_tensor if isinstance(acc, DTensor) else acc).add_(g)

    # ------------------------------------------------------------ state dict --
    def full_tensor(self) -> torch.Tensor:
        shard = self.sharded_local.data.to(self.device)
        if self.n == 1:
            return shard.clone()
        buf = torch.empty((self.n,) + tuple(shard.shape), dtype=shard.dtype, device=self.device)
        cc.all_gather_into(buf.view(self.n * shard.shape[0], *shard.shape[1:]), shard.contiguous(),
                           self.mesh_info.shard_group)
        return buf.movedim(0, self.shard_dim).reshape(self.full_shape)
