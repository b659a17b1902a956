"""Configuration objects of the HSDP engine
(hyper_parallel/core/hsdp/hsdp_utils.py:19-71 of the reference)."""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Optional, Tuple

import torch


class OptimizerLevel(enum.Enum):
    """What is sharded: level1 = optimizer state + weights, level2 = + gradients,
    level3 = + weights are re-gathered in backward (never kept unsharded between fwd and bwd)."""
    SHARD_OPT = "level1"
    SHARD_OPT_GRAD = "level2"
    SHARD_OPT_GRAD_PARAM = "level3"


@dataclass
class HSDPConfig:
    shard_size: int = -1
    threshold: int = 64 * 1024           # bytes; smaller parameters stay unsharded
    shard_level: OptimizerLevel = OptimizerLevel.SHARD_OPT
    requires_acc_grad: bool = False
    grad_scale: float = 1.0
    reduce_dtype: Optional[torch.dtype] = None
    comm_async: bool = False
    comm_fusion: bool = False
    bucket_size: int = -1                # bytes; -1 = one bucket per (groups, dtype)
    use_eager_hook: bool = True

    @property
    def grad_fusion(self) -> bool:
        return self.comm_fusion and self.bucket_size != 0


@dataclass
class GroupInfo:
    """A communication group: its ranks, the torch process group and this rank's index in it."""
    name: str
    ranks: Tuple[int, ...] = field(default_factory=tuple)
    group: object = None
    rank_size: int = 1
    index: int = 0
