"""Policies and mesh descriptors of ``fully_shard``
(hyper_parallel/platform/torch/fully_shard/utils.py:8-93 of the reference)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..device_mesh import DeviceMesh


@dataclass(frozen=True)
class MixedPrecisionPolicy:
    """``param_dtype``: dtype of the gathered (compute) parameters; ``reduce_dtype``: dtype of the
    gradient collectives; ``output_dtype``: cast of floating-point forward outputs;
    ``cast_forward_inputs``: cast floating-point forward inputs to ``param_dtype``;
    ``apply_grad_on_fp32_main_grad``: accumulate reduced gradients into an fp32 ``main_grad``
    attribute of the sharded parameter instead of ``.grad``."""
    param_dtype: Optional[torch.dtype] = None
    reduce_dtype: Optional[torch.dtype] = None
    output_dtype: Optional[torch.dtype] = None
    cast_forward_inputs: bool = True
    apply_grad_on_fp32_main_grad: bool = False


@dataclass
class OffloadPolicy:
    """No offloading."""


@dataclass
class CPUOffloadPolicy(OffloadPolicy):
    """Keep sharded parameters (and their gradients / optimizer state) in host memory."""
    pin_memory: bool = True


@dataclass
class DataParallelMeshInfo:
    mesh: DeviceMesh
    shard_mesh_dim: Optional[int] = None
    replicate_mesh_dim: Optional[int] = None

    def __post_init__(self):
        self.shard_group = self.mesh.get_group(self.shard_mesh_dim) if self.shard_mesh_dim is not None else None
        self.replicate_group = self.mesh.get_group(self.replicate_mesh_dim) \
            if self.replicate_mesh_dim is not None else None
        self.shard_size = self.mesh.size(self.shard_mesh_dim) if self.shard_mesh_dim is not None else 1
        self.replicate_size = self.mesh.size(self.replicate_mesh_dim) if self.replicate_mesh_dim is not None else 1
        self.shard_rank = self.mesh.get_local_rank(self.shard_mesh_dim) if self.shard_mesh_dim is not None else 0


class FSDPMeshInfo(DataParallelMeshInfo):
    """1-D mesh: shard over all of it."""

    def __init__(self, mesh: DeviceMesh, shard_mesh_dim: int = 0):
        super().__init__(mesh, shard_mesh_dim=shard_mesh_dim)


class DDPMeshInfo(DataParallelMeshInfo):
    """1-D mesh used for replication only."""

    def __init__(self, mesh: DeviceMesh, replicate_mesh_dim: int = 0):
        super().__init__(mesh, replicate_mesh_dim=replicate_mesh_dim)


class HSDPMeshInfo(DataParallelMeshInfo):
    """2-D mesh: replicate over dim 0, shard over dim 1."""

    def __init__(self, mesh: DeviceMesh, shard_mesh_dim: int = 1, replicate_mesh_dim: int = 0):
        super().__init__(mesh, shard_mesh_dim=shard_mesh_dim, replicate_mesh_dim=replicate_mesh_dim)


@dataclass
class StateDictOptions:
    """Same fields (and defaults) as ``torch.distributed.checkpoint.state_dict.StateDictOptions``, which
    the reference takes directly (hyper_parallel/core/fully_shard/api.py:443-490); an instance of the
    torch class is accepted wherever this one is."""
    full_state_dict: bool = False
    cpu_offload: bool = False
    ignore_frozen_params: bool = False
    keep_submodule_prefixes: bool = True
    strict: bool = True
    broadcast_from_rank0: bool = False
