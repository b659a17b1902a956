"""Per-parameter HSDP state: rank space, shard / replica groups, shard <-> unsharded data.

Rules follow hyper_parallel/core/hsdp/hsdp_param.py:21-308 and
hyper_parallel/platform/torch/hsdp/param.py:26-53 of the reference:

* HSDP works **on top of TP**: for a DTensor parameter the HSDP rank space is made
  of the mesh axes that do *not* shard it; for a plain parameter it is the world.
* ``shard_size = min(cfg or dim0, gcd(dim0_local, rank_size))``, reset to 1 when the
  gcd is not a multiple of it, when the parameter is smaller than ``threshold``
  bytes or has no dims; ``param.hsdp_shard_size`` overrides the configured value and
  the result is published as ``param.hsdp_effective_shard_size``.
* shard group = ``shard_size`` consecutive ranks of the space (all-gather /
  reduce-scatter), replica group = the ranks at stride ``shard_size`` (all-reduce).
* sharding is along **dim 0 of the local (TP-sharded) tensor**.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from ...collectives import cc
from ..dtensor import DTensor
from .hsdp_utils import GroupInfo, HSDPConfig, OptimizerLevel


class HSDPParam:
    def __init__(self, name: str, param: torch.nn.Parameter, config: HSDPConfig):
        self.name = name
        self.param = param
        self.config = config
        self.is_dtensor = isinstance(param, DTensor)
        self.acc_grad: Optional[torch.Tensor] = None
        self.reduced_grad: Optional[torch.Tensor] = None
        self.prefetch_handle = None
        self._unsharded_persistent: Optional[torch.Tensor] = None
        self.grad_ready = False
        self.grad_consumer = None   # optional callable(hp, reduced_grad) run as soon as the grad exists
        self._init_rank_space()
        self._init_shard_size()
        self._init_groups()
        self.sharded = self.shard_size > 1
        self.fully_sharded = self.sharded and self.dp_size == 1
        self.is_sharded_now = False
        self.full_shape = tuple(self.leaf.shape)
        self._shard_data()
        param._hsdp_param = self

    # the autograd leaf that actually holds data / grad
    @property
    def leaf(self) -> torch.Tensor:
        return self.param._local_tensor if self.is_dtensor else self.param

    # ------------------------------------------------------------ set-up --
    def _init_rank_space(self) -> None:
        me = cc.get_rank()
        if self.is_dtensor:
            layout = self.param.layout
            mesh = layout.mesh
            used = set(layout.sharded_axes)
            # axes over which the owner already synchronises this parameter's gradient itself
            # (e.g. tensor-parallel replicas whose gradients are all-reduced inside the TP region)
            for name in getattr(self.param, "hsdp_exclude_axes", ()):
                used.add(mesh._dim_index(name))
            coord = mesh.get_coordinate()
            if coord is None:
                raise RuntimeError(f"rank {me} is not in the mesh of parameter {self.name}")
            idx = tuple(slice(None) if a not in used else coord[a] for a in range(mesh.ndim))
            self.rank_list: List[int] = [int(r) for r in mesh._mesh[idx].reshape(-1)]
        else:
            self.rank_list = list(range(cc.get_world_size()))
        self.rank_size = len(self.rank_list)
        self.hsdp_rank = self.rank_list.index(me) if me in self.rank_list else 0

    def _init_shard_size(self) -> None:
        p, cfg = self.param, self.config
        ss = cfg.shard_size
        if hasattr(p, "hsdp_shard_size"):
            v = p.hsdp_shard_size
            if not isinstance(v, int) or (v <= 0 and v != -1):
                raise ValueError(f"param's hsdp_shard_size must be a positive integer, but got {v}.")
            ss = v
        local_shape = tuple(self.leaf.shape)
        if len(local_shape) < 1 or self.rank_size == 1:
            ss = 1
        else:
            nbytes = self.leaf.element_size() * math.prod(local_shape)
            if nbytes < cfg.threshold:
                ss = 1
            else:
                if ss == -1 or local_shape[0] < ss:
                    ss = local_shape[0]
                g = math.gcd(local_shape[0], self.rank_size)
                ss = min(ss, g)
                if ss <= 0 or g % ss != 0:
                    ss = 1
        self.shard_size = ss
        self.dp_size = self.rank_size // ss
        try:
            p.hsdp_effective_shard_size = ss
        except AttributeError:
            pass

    def _init_groups(self) -> None:
        ss, r = self.shard_size, self.hsdp_rank
        base = (r // ss) * ss
        shard_ranks = tuple(self.rank_list[base:base + ss])
        replica_ranks = tuple(self.rank_list[r % ss::ss])
        self.sharded_group_info = GroupInfo(
            "hsdp_sharded_dp_group_" + "_".join(map(str, shard_ranks)), shard_ranks,
            cc.group_for_ranks(shard_ranks) if ss > 1 else None, ss, r % ss)
        self.unsharded_group_info = GroupInfo(
            "hsdp_unsharded_dp_group_" + "_".join(map(str, replica_ranks)), replica_ranks,
            cc.group_for_ranks(replica_ranks) if self.dp_size > 1 else None, self.dp_size, r // ss)

    def _shard_data(self) -> None:
        if not self.sharded:
            self.shard = self.leaf.data
            return
        full = self.leaf.data
        if full.device.type == "meta":
            shape = (full.shape[0] // self.shard_size,) + tuple(full.shape[1:])
            self.shard = torch.empty(shape, dtype=full.dtype, device="meta")
        else:
            self.shard = full.chunk(self.shard_size, dim=0)[self.sharded_group_info.index].clone()
        self.leaf.data = self.shard
        self.is_sharded_now = True

    def rebind_param(self, new_param: torch.nn.Parameter) -> None:
        """Follow a parameter object that was re-created (meta -> real materialisation)."""
        self.param = new_param
        self.is_dtensor = isinstance(new_param, DTensor)
        new_param._hsdp_param = self
        self.shard = self.leaf.data
        self.is_sharded_now = self.sharded
        self._unsharded_persistent = None
        self.prefetch_handle = None
        try:
            new_param.hsdp_effective_shard_size = self.shard_size
        except AttributeError:
            pass
        hook = getattr(self, "_grad_hook_fn", None)
        if hook is not None and new_param.requires_grad:
            self.leaf.register_post_accumulate_grad_hook(hook)

    @property
    def shard_shape(self):
        if not self.sharded:
            return self.full_shape
        return (self.full_shape[0] // self.shard_size,) + self.full_shape[1:]

    def rebind_shard(self, new_shard: torch.Tensor) -> None:
        """Make ``new_shard`` (e.g. a view of a flat buffer) the storage of the sharded parameter."""
        self.shard = new_shard
        if self.is_sharded_now or not self.sharded:
            self.leaf.data = new_shard

    # ------------------------------------------------------- (un)sharding --
    def _full_buffer(self) -> torch.Tensor:
        keep = self.config.shard_level != OptimizerLevel.SHARD_OPT_GRAD_PARAM
        if keep and self._unsharded_persistent is not None:
            return self._unsharded_persistent
        buf = torch.empty(self.full_shape, dtype=self.shard.dtype, device=self.shard.device)
        if keep:
            self._unsharded_persistent = buf
        return buf

    def prefetch_unsharded(self) -> None:
        """Start an asynchronous all-gather of this parameter."""
        if not self.sharded or not self.is_sharded_now or self.prefetch_handle is not None:
            return
        buf = self._full_buffer()
        work = cc.all_gather_into(buf, self.shard, self.sharded_group_info.group, async_op=True)
        self.prefetch_handle = (work, buf)

    def to_unsharded(self) -> None:
        if not self.sharded or not self.is_sharded_now:
            return
        if self.prefetch_handle is not None:
            work, buf = self.prefetch_handle
            self.prefetch_handle = None
            if work is not None:
                work.wait()
        else:
            buf = self._full_buffer()
            cc.all_gather_into(buf, self.shard, self.sharded_group_info.group)
        self.leaf.data = buf
        self.is_sharded_now = False

    def to_sharded(self) -> None:
        if not self.sharded or self.is_sharded_now:
            return
        self.leaf.data = self.shard
        self.is_sharded_now = True

    # ---------------------------------------------------- grad accumulation --
    def ensure_acc_grad(self, like: torch.Tensor) -> torch.Tensor:
        if self.acc_grad is None or self.acc_grad.shape != like.shape:
            self.acc_grad = torch.zeros_like(like)
        return self.acc_grad

    def zero_acc_grad(self) -> None:
        if self.acc_grad is not None:
            self.acc_grad.zero_()
